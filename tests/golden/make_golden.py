"""Generates the committed fixtures of tests/golden/ from the CPU oracle (oracle/ref.py, cross-checked
against oracle/fp8_oracle.c while generating).

    python tests/golden/make_golden.py

The reference ships no golden vectors for this path, so these fixtures pin the repository's own
restatement (regression pins, "parity unpinned"): a table of e4m3 round-to-nearest-even edge cases, one
small quantize + GEMM case stored in full, and checksums of the CPU-runnable configuration
(M=256, N=1024, K=1024, seed 0).
"""
import hashlib
import json
import os
import struct
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import cref, ref  # noqa: E402


def f32_hex(v: float) -> str:
    return struct.pack(">f", v).hex()


def sha(t: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def edge_cases():
    vals = [0.0, -0.0, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -9, 2.5 * 2.0 ** -9, 3.5 * 2.0 ** -9, 7.5 * 2.0 ** -9,
            2.0 ** -6, 2.0 ** -6 * 1.0625, 2.0 ** -6 * 1.1875, 1.0, 1.0625, 1.1875, 17.0, 18.0, 19.0, 240.0, 416.0, 432.0,
            440.0, 448.0, 448.00003, 463.9, 464.0, 464.1, 480.0, 1e9, -17.0, -448.0, -464.0, -465.0, 1e-30, -1e-30]
    rows = []
    for v in vals:
        v32 = float(np.float32(v))
        t = torch.tensor([v32], dtype=torch.float32).to(torch.float8_e4m3fn).view(torch.uint8).item()
        c_nonsat = cref.e4m3_encode(v32, saturate=False)
        c_sat = cref.e4m3_encode(v32, saturate=True)
        assert t == c_nonsat, (v32, t, c_nonsat)
        rows.append({"f32": f32_hex(v32), "value": v32, "code_torch_nonsat": int(t), "code_satfinite": int(c_sat)})
    decode = [None if (c & 0x7f) == 0x7f else cref.e4m3_decode(c) for c in range(256)]
    return {"encode": rows, "decode_table": decode}


def small_case():
    g = torch.Generator().manual_seed(1234)
    m, n, k = 128, 256, 256
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    a[0, :128] = 0                      # all-zero group: amax floor
    a[1, :128] = torch.arange(128) - 64  # hand-checkable: amax 64 -> scale 64/448 = 1/7
    a[2, 128:] = 448.0                  # scale exactly 1, every code 0x7e
    b = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    qa, sa = ref.per_token_cast_to_fp8(a)
    qb, sb = ref.per_block_cast_to_fp8(b)
    qa_c, sa_c = cref.per_token_cast_to_fp8(a.view(torch.uint16).numpy())
    qb_c, sb_c = cref.per_block_cast_to_fp8(b.view(torch.uint16).numpy())
    assert np.array_equal(qa.view(torch.uint8).numpy(), qa_c) and np.array_equal(sa.t().contiguous().numpy(), sa_c)
    assert np.array_equal(qb.view(torch.uint8).numpy(), qb_c) and np.array_equal(sb.numpy(), sb_c)
    d = ref.ref_gemm((qa, sa), (qb, sb))
    np.savez_compressed(os.path.join(HERE, "small_128x256x256.npz"),
                        a_bf16=a.view(torch.uint16).numpy(), b_bf16=b.view(torch.uint16).numpy(),
                        qa=qa.view(torch.uint8).numpy(), sa_kmajor=sa.t().contiguous().numpy(),
                        qb=qb.view(torch.uint8).numpy(), sb=sb.numpy(), d_bf16=d.view(torch.uint16).numpy())


def config1_checksums():
    a, b = ref.make_inputs(256, 1024, 1024, seed=0)
    qa, sa = ref.per_token_cast_to_fp8(a)
    qb, sb = ref.per_block_cast_to_fp8(b)
    d = ref.ref_gemm((qa, sa), (qb, sb)).float()
    return {"shape": [256, 1024, 1024], "seed": 0,
            "a_bf16_sha256": sha(a.view(torch.uint16).numpy()), "b_bf16_sha256": sha(b.view(torch.uint16).numpy()),
            "qa_sha256": sha(qa.view(torch.uint8).numpy()), "sa_kmajor_sha256": sha(sa.t().contiguous().numpy()),
            "qb_sha256": sha(qb.view(torch.uint8).numpy()), "sb_sha256": sha(sb.numpy()),
            "d_rms": float(d.pow(2).mean().sqrt()), "d_absmax": float(d.abs().max()), "d_sum": float(d.double().sum()),
            "d_probe": {"[0,0]": float(d[0, 0]), "[17,301]": float(d[17, 301]), "[255,1023]": float(d[255, 1023])}}


if __name__ == "__main__":
    with open(os.path.join(HERE, "e4m3_edge_cases.json"), "w") as f:
        json.dump(edge_cases(), f, indent=1)
    small_case()
    with open(os.path.join(HERE, "config1_checksums.json"), "w") as f:
        json.dump(config1_checksums(), f, indent=1)
    print("fixtures written to", HERE)
