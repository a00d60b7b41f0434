#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference's own CPU code.

Run once on a machine that has the reference checkout:

    python tests/golden/make_golden.py --reference <path-to-reference-checkout>

The script executes the *reference's* CPU helpers (it extracts the function
definitions from the reference's test and benchmark scripts with ``ast`` so
that their module-level GPU imports and prints do not run) on the reference's
own seeds and shapes, and stores inputs/outputs as small ``.npz`` files.
Nothing here is needed at test time; the tests read only the ``.npz`` files.

Vectors written
---------------
kat_gemm_4x128x8.npz       int4_native_tc/test_correctness.py:131-157 (seed 42)
kat_gemm_16x2560x2560.npz  int4_native_tc/test_correctness.py:164-186 (seed 123; inputs
                           regenerated from the seed at test time, output stored)
kat_unpack_16x256.npz      int4_native_tc/test_correctness.py:653-674 (seed 99)
kat_scaled_8x256x16.npz    int4_native_tc/test_correctness.py:193-221 (seed 77; the
                           reference draws its scales from the unseeded global RNG, so the
                           scales stored here come from RandomState(78))
kat_native_matmul.npz      benchmark/verify_int4_matmul_precision.py:16-29 (int32 torch matmul
                           followed by fp32 scales) on a 16x512x64 case
kat_quant_formula.npz      benchmark/benchmark_w4a8fp8.py:200-204 per-group weight quantiser
                           formula applied to a 32x512 bf16 matrix
kat_w4a8_8x256x64.npz      int4_native_tc/test_correctness.py:551-566 (seed 88): int8 activations x int4
                           weights, the int32 product and the scaled fp32 reference of the test's own CPU
                           lines (executed from the reference file); scales from RandomState(89)
"""
from __future__ import annotations

import argparse
import ast
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_functions(path: str, names: list[str], extra_globals: dict | None = None) -> dict:
    """Compile only the named top-level function definitions of a Python file."""
    with open(path, "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in keep}
    if missing:
        raise RuntimeError(f"{path}: functions not found: {sorted(missing)}")
    mod = ast.Module(body=keep, type_ignores=[])
    env = {"np": np, "torch": torch}
    env.update(extra_globals or {})
    exec(compile(mod, path, "exec"), env)
    return {n: env[n] for n in names}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the reference checkout")
    args = ap.parse_args()
    ref = args.reference

    tc = load_functions(
        os.path.join(ref, "int4_native_tc", "test_correctness.py"),
        ["pack_int4_cpu", "unpack_int4_cpu", "int4_gemm_cpu"],
    )
    vp = load_functions(
        os.path.join(ref, "benchmark", "verify_int4_matmul_precision.py"),
        ["int4_native_matmul"],
    )
    pack, unpack, gemm = tc["pack_int4_cpu"], tc["unpack_int4_cpu"], tc["int4_gemm_cpu"]

    # -- integer GEMM KATs (the reference's seeds and shapes) -------------------
    rng = np.random.RandomState(42)
    a = rng.randint(-8, 8, size=(4, 128)).astype(np.int8)
    b = rng.randint(-8, 8, size=(8, 128)).astype(np.int8)
    np.savez_compressed(
        os.path.join(HERE, "kat_gemm_4x128x8.npz"),
        a=a, b=b, a_packed=pack(a), b_packed=pack(b), c=gemm(a, b),
    )

    rng = np.random.RandomState(123)
    a = rng.randint(-8, 8, size=(16, 2560)).astype(np.int8)
    b = rng.randint(-8, 8, size=(2560, 2560)).astype(np.int8)
    np.savez_compressed(
        os.path.join(HERE, "kat_gemm_16x2560x2560.npz"),
        seed=np.int64(123), c=gemm(a, b), a_packed_row0=pack(a[:1]), b_packed_row0=pack(b[:1]),
    )

    # -- unpack round trip ------------------------------------------------------
    rng = np.random.RandomState(99)
    w = rng.randint(-8, 8, size=(16, 256)).astype(np.int8)
    wp = pack(w)
    np.savez_compressed(
        os.path.join(HERE, "kat_unpack_16x256.npz"), codes=w, packed=wp, unpacked=unpack(wp, 256)
    )

    # -- scaled epilogue ---------------------------------------------------------
    rng = np.random.RandomState(77)
    a = rng.randint(-8, 8, size=(8, 256)).astype(np.int8)
    b = rng.randint(-8, 8, size=(16, 256)).astype(np.int8)
    srng = np.random.RandomState(78)
    sa = srng.rand(8).astype(np.float32) * 0.1
    sb = srng.rand(16).astype(np.float32) * 0.1
    acc = gemm(a, b).astype(np.float32)
    np.savez_compressed(
        os.path.join(HERE, "kat_scaled_8x256x16.npz"),
        a=a, b=b, scale_a=sa, scale_b=sb, ref=acc * sa[:, None] * sb[None, :],
    )

    # -- the reference's torch "native" path --------------------------------------
    g = torch.Generator().manual_seed(5)
    A = torch.randint(-8, 8, (16, 512), generator=g, dtype=torch.int8)
    B = torch.randint(-8, 8, (64, 512), generator=g, dtype=torch.int8)
    sA = torch.rand(16, generator=g) * 0.1
    sB = torch.rand(64, generator=g) * 0.1
    out = vp["int4_native_matmul"](A, B, sA, sB)
    np.savez_compressed(
        os.path.join(HERE, "kat_native_matmul.npz"),
        a=A.numpy(), b=B.numpy(), scale_a=sA.numpy(), scale_b=sB.numpy(), ref=out.numpy(),
    )

    # -- quantiser formula, as written at benchmark/benchmark_w4a8fp8.py:200-204 ---
    g = torch.Generator().manual_seed(6)
    w_bf16 = (torch.randn(32, 512, generator=g) * 0.02).to(torch.bfloat16)
    N, K, GS = 32, 512, 128
    w_fp32 = w_bf16.float()
    w_reshaped = w_fp32.reshape(N, K // GS, GS)
    g_amax = w_reshaped.abs().amax(dim=2).clamp(min=1e-12)
    g_scale = g_amax / 7.0
    w_int4 = torch.clamp(torch.round(w_reshaped / g_scale.unsqueeze(2)), -8, 7)
    np.savez_compressed(
        os.path.join(HERE, "kat_quant_formula.npz"),
        w_bf16_bits=w_bf16.view(torch.int16).numpy(),
        codes=w_int4.to(torch.int8).numpy(),  # [N, G, GS]
        scale=g_scale.numpy(),  # [N, G]
    )
    # -- W4A8: the CPU lines of the reference's own test, executed from its source ------------------------
    src = open(os.path.join(ref, "int4_native_tc", "test_correctness.py"), encoding="utf-8").read().splitlines()
    body = [ln.strip() for ln in src[552:566]]          # test_w4a8_scaled_gemm: inputs and CPU reference
    wanted = [ln for ln in body if ln.startswith(("M, K, N", "rng =", "a_int8 =", "b_int4 =", "acc =", "ref ="))]
    env = {"np": np}
    srng = np.random.RandomState(89)
    for ln in wanted:
        if ln.startswith("acc ="):
            env["scale_a"] = srng.rand(env["M"]).astype(np.float32) * 0.01
            env["scale_b"] = srng.rand(env["N"]).astype(np.float32) * 0.1
        exec(ln, env)
    np.savez_compressed(
        os.path.join(HERE, "kat_w4a8_8x256x64.npz"),
        a=env["a_int8"], b=env["b_int4"], scale_a=env["scale_a"], scale_b=env["scale_b"], acc=env["acc"], ref=env["ref"],
    )
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
