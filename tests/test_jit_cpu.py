"""CPU tests of the JIT layer: code generation (string level), type maps, cache layout and a compile-only
build for sm_100a (nvcc cross-compiles without a GPU).  Mirrors what the reference's tests/test_jit.py checks
up to the point where a GPU is needed."""
import os

import pytest
import torch

from yan_b200 import jit
from yan_b200.jit import template as T

ARGS = (('lhs', torch.float8_e4m3fn), ('rhs', torch.float8_e4m3fn), ('scale', torch.float), ('out', torch.bfloat16),
        ('enable_double_streams', bool), ('stream', torch.cuda.Stream))


def test_generate_signature_and_casts():
    code = jit.generate((), ARGS, "int x = 0;\n")
    assert ('extern "C" EXPORT_API void launch(void* __raw_lhs, void* __raw_rhs, void* __raw_scale, void* __raw_out, '
            'bool enable_double_streams, void* __raw_stream, int& __return_code)') in code
    assert "auto lhs = reinterpret_cast<__nv_fp8_e4m3*>(__raw_lhs);" in code
    assert "auto scale = reinterpret_cast<float*>(__raw_scale);" in code
    assert "auto out = reinterpret_cast<__nv_bfloat16*>(__raw_out);" in code
    assert "auto stream = reinterpret_cast<cudaStream_t>(__raw_stream);" in code
    assert "__raw_enable_double_streams" not in code
    for inc in ("<cuda.h>", "<cuda_fp8.h>", "<cuda_runtime.h>", "<iostream>"):
        assert f"#include {inc}" in code


def test_generate_includes_are_sorted_and_deduplicated():
    code = jit.generate(('"gemm/fp8_gemm.cuh"', '<vector>', '"gemm/fp8_gemm.cuh"'), (('m', int),), "")
    assert code.count('#include "gemm/fp8_gemm.cuh"') == 1 and "#include <vector>" in code
    assert code.index("#include <cuda.h>") < code.index("#include <vector>") < code.index('#include "gemm/fp8_gemm.cuh"')


def test_cpp_format_leaves_other_braces_alone():
    out = jit.cpp_format("constexpr auto N = {N}; struct S { int a{K}; };", {"N": 4096, "K": 7})
    assert out == "constexpr auto N = 4096; struct S { int a7; };"
    assert jit.cpp_format("void f() { g({X}); }", {"X": "1"}) == "void f() { g(1); }"


def test_type_maps_cover_the_reference_types():
    for t in (bool, int, float, torch.int, torch.float, torch.half, torch.bfloat16, torch.float8_e4m3fn, torch.cuda.Stream):
        assert t in T.typename_map and t in T.ctype_map and t in T.genc_map
    assert T.genc_map[torch.float8_e4m3fn] == ("void*", "__nv_fp8_e4m3*")
    assert T.map_ctype(3).value == 3 and T.map_ctype(True).value is True
    x = torch.zeros(4)
    assert T.map_ctype(x).value == x.data_ptr()


def test_fp8_gemm_template_keeps_the_reference_variable_names():
    from yan_b200.jit_kernels import gemm
    for token in ("{N}", "{K}", "{BLOCK_M}", "{BLOCK_N}", "{NUM_STAGES}", "make_2d_tma_a_desc(lhs, m)",
                  "make_2d_tma_b_desc(rhs)", "make_2d_tma_scales_a_desc(lhs_scales, m)", "make_2d_tma_d_desc(out, m)",
                  "GemmType::run(out, rhs_scales, nullptr", "stream, num_sms, smem_size"):
        assert token in gemm.template
    names = [n for n, _ in gemm.arg_defs]
    assert names == ['lhs', 'lhs_scales', 'rhs', 'rhs_scales', 'out', 'm', 'stream', 'num_sms', 'smem_size']


def test_arch_flag_targets_sm_100a_without_a_gpu(monkeypatch):
    from yan_b200.jit import compiler
    if torch.cuda.is_available():
        pytest.skip("CPU-only check")
    monkeypatch.delenv("YAN_JIT_ARCH", raising=False)
    assert compiler.get_arch_flag() == "-gencode=arch=compute_100a,code=sm_100a"
    assert "--use_fast_math" not in compiler.get_flags()


def test_build_compiles_and_caches(tmp_path, monkeypatch):
    from yan_b200.jit import compiler
    monkeypatch.setenv("YAN_CACHE_DIR", str(tmp_path))
    compiler.get_default_user_dir.cache_clear()
    try:
        code = jit.generate((), ARGS, "__return_code = enable_double_streams ? 0 : 3;\n")
        rt = jit.build("cpu_build_check", ARGS, code)
        assert os.path.basename(rt.path).startswith("kernel.cpu_build_check.") and str(tmp_path) in rt.path
        for f in ("kernel.cu", "kernel.args", "kernel.so"):
            assert os.path.exists(os.path.join(rt.path, f))
        assert eval(open(os.path.join(rt.path, "kernel.args")).read(), {"torch": torch}) == ARGS
        assert jit.build("cpu_build_check", ARGS, code) is rt          # memoised
        other = jit.build("cpu_build_check", ARGS, code + "// changed\n")
        assert other.path != rt.path                                    # hash covers the code
    finally:
        compiler.get_default_user_dir.cache_clear()


def test_fp8_gemm_template_cross_compiles(tmp_path, monkeypatch):
    from yan_b200.jit import compiler
    from yan_b200.jit_kernels import gemm
    monkeypatch.setenv("YAN_CACHE_DIR", str(tmp_path))
    compiler.get_default_user_dir.cache_clear()
    try:
        keys = {'N': 1024, 'K': 1024, 'BLOCK_M': 128, 'BLOCK_N': 64, 'NUM_STAGES': 8}
        code = jit.generate(gemm.includes, gemm.arg_defs, jit.cpp_format(gemm.template, keys))
        rt = jit.build("gemm_fp8_fp8_bf16_nt", gemm.arg_defs, code)
        assert os.path.exists(os.path.join(rt.path, "kernel.so"))
    finally:
        compiler.get_default_user_dir.cache_clear()


def test_best_config_heuristic():
    from yan_b200.jit_kernels import gemm
    assert gemm.get_best_configs(8192, 28672, 8192, 148)[0] == 256
    assert gemm.get_best_configs(4096, 7168, 18432, 148)[0] == 256
    bn, stages, smem = gemm.get_best_configs(16, 7168, 2048, 148)
    assert bn in (32, 64, 128) and smem <= 232448
    for bn, st in gemm._DEFAULT_STAGES.items():
        assert gemm.get_smem_size(bn, st) <= 232448


def test_host_utils():
    from yan_b200.jit_kernels import utils
    assert utils.ceil_div(7, 2) == 4 and utils.get_m_alignment_for_contiguous_layout() == 128
    x = torch.arange(12.0).view(3, 4)
    c = utils.get_col_major_tensor(x)
    assert c.shape == (3, 4) and c.stride() == (1, 3) and torch.equal(c, x)
    assert utils.get_col_major_tensor(c).data_ptr() == c.data_ptr()  # already column-major: no copy
    from yan_b200 import utils as U
    assert abs(float(U.calc_diff(x, x))) < 1e-12 and U.count_bytes((x, (x, x))) == 3 * 48


def test_perf_log_appends_json_lines(tmp_path, monkeypatch):
    import json
    from yan_b200.utils import perf_log
    path = tmp_path / "perf.jsonl"
    perf_log({"workload": "ignored: no file named"})
    monkeypatch.setenv("YAN_PERF_LOG", str(path))
    perf_log({"workload": "C1", "us": 10.5, "TFLOP/s": 51.0})
    perf_log({"workload": "C2", "us": 5.4, "GB/s": 2750.0})
    lines = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["workload"] for r in lines] == ["C1", "C2"] and lines[0]["us"] == 10.5 and "unix_time" in lines[1]
