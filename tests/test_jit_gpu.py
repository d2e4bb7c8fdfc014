"""GPU tests of the JIT route: the reference's own JIT conformance check (tests/test_jit.py:37-62 -- generated
stub prints its arguments, return code 0, stdout equals the pointer values) and the FP8 template compiled and
run through compile_and_tune."""
import os

import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


class Capture:
    def __enter__(self):
        self.read_fd, self.write_fd = os.pipe()
        self.saved_stdout = os.dup(1)
        os.dup2(self.write_fd, 1)
        return self

    def __exit__(self, *exc):
        os.dup2(self.saved_stdout, 1)
        os.close(self.write_fd)
        with os.fdopen(self.read_fd, "r") as f:
            self.captured = f.read()


def test_jit_stub_receives_pointers_and_flags(cuda_lib, tmp_path, monkeypatch):
    from yan_b200 import jit
    from yan_b200.jit import compiler
    monkeypatch.setenv("YAN_CACHE_DIR", str(tmp_path))
    compiler.get_default_user_dir.cache_clear()
    try:
        args = (('lhs', torch.float8_e4m3fn), ('rhs', torch.float8_e4m3fn), ('scale', torch.float),
                ('out', torch.bfloat16), ('enable_double_streams', bool), ('stream', torch.cuda.Stream))
        body = "\n"
        for name in ("lhs", "rhs", "scale", "out"):
            body += f"std::cout << reinterpret_cast<uint64_t>({name}) << std::endl;\n"
        body += "std::cout << enable_double_streams << std::endl;\n"
        body += "std::cout << reinterpret_cast<uint64_t>(stream) << std::endl;\n"
        func = jit.build("test_func", args, jit.generate((), args, body))
        fp8 = torch.empty((1,), dtype=torch.float8_e4m3fn, device="cuda")
        fp32 = torch.empty((1,), dtype=torch.float, device="cuda")
        bf16 = torch.empty((1,), dtype=torch.bfloat16, device="cuda")
        stream = torch.cuda.current_stream()
        with Capture() as cap:
            assert func(fp8, fp8, fp32, bf16, True, stream) == 0
        expected = f"{fp8.data_ptr()}\n{fp8.data_ptr()}\n{fp32.data_ptr()}\n{bf16.data_ptr()}\n1\n{stream.cuda_stream}\n"
        assert cap.captured == expected
        with pytest.raises(AssertionError):
            func(fp32, fp8, fp32, bf16, True, stream)       # dtype mismatch is caught before the call
    finally:
        compiler.get_default_user_dir.cache_clear()


def test_fp8_gemm_through_jit_template(cuda_lib, tmp_path, monkeypatch):
    import yan_b200
    from yan_b200.jit import compiler
    monkeypatch.setenv("YAN_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("YAN_FP8_GEMM_JIT", "1")
    compiler.get_default_user_dir.cache_clear()
    try:
        a, b = ref.make_inputs(256, 1024, 1024, seed=0)
        lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
        out = torch.empty(256, 1024, dtype=torch.bfloat16, device="cuda")
        yan_b200.gemm_fp8_fp8_bf16_nt((lhs[0].cuda(), lhs[1].t().contiguous().cuda().t()), (rhs[0].cuda(), rhs[1].cuda()),
                                      out, block_n=128)
        torch.cuda.synchronize()
        assert ref.rel_frobenius(out.cpu(), ref.ref_gemm(lhs, rhs)) <= 1e-3
        assert any(d.startswith("kernel.gemm_fp8_fp8_bf16_nt.") for d in os.listdir(os.path.join(tmp_path, "cache")))
        # the JIT-compiled library has a status word of its own, which the package-level read covers
        from yan_b200.jit_kernels import gemm as gemm_module
        used = [r for r in gemm_module._jit_runtimes_used.values() if str(tmp_path) in r.path]
        assert used and hasattr(used[0].lib, "yan_jit_read_device_status")
        assert used[0].read_device_status() == 0 and yan_b200.read_device_status() == 0
    finally:
        compiler.get_default_user_dir.cache_clear()


def test_bench_kineto_finds_the_gemm_kernel(cuda_lib):
    import yan_b200
    a, b = ref.make_inputs(256, 1024, 1024, seed=0)
    lhs = yan_b200.per_token_cast_to_fp8(a.cuda())
    rhs = yan_b200.per_block_cast_to_fp8(b.cuda())
    out = torch.empty(256, 1024, dtype=torch.bfloat16, device="cuda")
    t = yan_b200.bench_kineto(lambda: yan_b200.gemm_fp8_fp8_bf16_nt(lhs, rhs, out), "fp8_gemm_kernel", num_tests=5,
                              suppress_kineto_output=True)
    assert 0 < t < 1e-3


def test_tuner_times_a_space_and_remembers_the_winner(cuda_lib, tmp_path, monkeypatch):
    """compile_and_tune over several tile widths: every candidate is built, launched (non-zero return codes are
    skipped), timed, and the winner is stored in tuned.json so that a new tuner does not time again."""
    import json
    import yan_b200
    from yan_b200.jit import compiler
    from yan_b200.jit_kernels.tuner import JITTuner
    monkeypatch.setenv("YAN_CACHE_DIR", str(tmp_path))
    monkeypatch.setenv("YAN_FP8_GEMM_JIT", "1")
    monkeypatch.setenv("YAN_FP8_GEMM_TUNE", "1")
    compiler.get_default_user_dir.cache_clear()
    try:
        a, b = ref.make_inputs(128, 128, 512, seed=2)      # N = 128: the space is BLOCK_N in {128, 96, 64, 32}
        lhs, rhs = ref.per_token_cast_to_fp8(a), ref.per_block_cast_to_fp8(b)
        out = torch.empty(128, 128, dtype=torch.bfloat16, device="cuda")
        yan_b200.gemm_fp8_fp8_bf16_nt((lhs[0].cuda(), lhs[1].t().contiguous().cuda().t()), (rhs[0].cuda(), rhs[1].cuda()), out)
        torch.cuda.synchronize()
        assert ref.rel_frobenius(out.cpu(), ref.ref_gemm(lhs, rhs)) <= 1e-3
        built = [d for d in os.listdir(os.path.join(tmp_path, "cache")) if d.startswith("kernel.gemm_fp8_fp8_bf16_nt.")]
        assert len(built) == 4
        with open(os.path.join(tmp_path, "cache", "tuned.json")) as f:
            stored = json.load(f)
        assert len(stored) == 1 and list(stored.values())[0]["BLOCK_N"] in (128, 96, 64, 32)
        # a fresh tuner (new process in real life) goes straight to the remembered configuration
        fresh = JITTuner()
        assert fresh._load_choice(list(stored.keys())[0]) == list(stored.values())[0]
    finally:
        compiler.get_default_user_dir.cache_clear()
