#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference's own Python functions.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/reference

The reference modules cannot be imported as a whole (they import packages that are not part
of the repository at module scope), so the functions named below are lifted out of their
files by name with `ast` and executed unmodified against torch.  Only their OUTPUTS are
written here; no reference source is stored.

  select params ........... tools/bench_qwen3_l18_split_opts_v57.py        split_select_params
  R from ratio ............ tools/bench_v61_dense_sparse_matrix_breakdown_v1.py  ceil_ratio_count
  thresholds + indices .... tools/bench_topr_select_algos_v38.py           current_select
                            tools/compare_single_matrix_fake_vs_kernel_quant_l2_v1.py  compute_thresholds_and_indices
  fake quant .............. tools/compare_single_matrix_fake_vs_kernel_quant_l2_v1.py  fake_quant_reconstruct, decode_signed_int4
  RTN weight scale ........ tools/bench_multimodel_all_layers_policy_fastqf_v29.py  make_rtn_scale_cpu
  RTN weight codes ........ tools/bench_real_split_fullstack_rtn_ppl_v1.py   rtn_quantize_with_scale
  policy loader ........... tools/bench_multimodel_all_layers_policy_fastqf_v29.py  load_policy, normalize_name

torch.topk does not define the order of equal keys, so the select inputs are built with
pairwise distinct magnitudes; the tie rule itself (lowest index first) is taken from
reading tools/fused_threshold_topr_pack_ext_v57.py:141-181 and is tested separately.
"""
from __future__ import annotations

import argparse
import ast
import json
import math
import types
from pathlib import Path

import numpy as np
import torch


def lift(path: Path, names, extra_globals=None):
    """Compile the named top-level functions of a file, nothing else."""
    tree = ast.parse(path.read_text(encoding="utf-8"))
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in body}
    if missing:
        raise RuntimeError(f"{path}: missing {missing}")
    mod = ast.Module(body=body, type_ignores=[])
    g = {"torch": torch, "math": math, "json": json, "Path": Path, "__builtins__": __builtins__}
    g.update(extra_globals or {})
    exec(compile(mod, str(path), "exec"), g)
    return types.SimpleNamespace(**{n: g[n] for n in names})


def distinct_rows(M: int, K: int, seed: int) -> np.ndarray:
    """bf16-representable rows whose magnitudes are pairwise distinct within a row."""
    rng = np.random.default_rng(seed)
    # all positive bf16 patterns in a band of exponents: 128 mantissas per binade
    n_binades = (K + 127) // 128 + 2
    base = 0x3F80 - 128 * (n_binades // 2)
    pool = np.arange(base, base + 128 * n_binades, dtype=np.uint16)
    out = np.empty((M, K), dtype=np.uint16)
    for m in range(M):
        mags = rng.permutation(pool)[:K]
        signs = rng.integers(0, 2, K).astype(np.uint16) << np.uint16(15)
        out[m] = mags | signs
    return out


def bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent))
    args = ap.parse_args()
    ref = Path(args.reference) / "tools"
    out = Path(args.out)

    v57 = lift(ref / "bench_qwen3_l18_split_opts_v57.py", ["split_select_params"])
    v61 = lift(ref / "bench_v61_dense_sparse_matrix_breakdown_v1.py", ["ceil_ratio_count"])
    v38 = lift(ref / "bench_topr_select_algos_v38.py", ["current_select"])
    cmp_ = lift(ref / "compare_single_matrix_fake_vs_kernel_quant_l2_v1.py",
                ["compute_thresholds_and_indices", "fake_quant_reconstruct", "decode_signed_int4"])
    v29 = lift(ref / "bench_multimodel_all_layers_policy_fastqf_v29.py",
               ["make_rtn_scale_cpu", "load_policy", "normalize_name"])
    rtn = lift(ref / "bench_real_split_fullstack_rtn_ppl_v1.py", ["rtn_quantize_with_scale"])

    # ---- scalars -----------------------------------------------------------------
    scalars = []
    for K in (64, 128, 4096, 12288, 14336):
        for ratio in (0.0, 0.0025, 0.01, 0.05, 0.10, 0.999, 1.5):
            R = int(v61.ceil_ratio_count(K, ratio))
            for pct in (100.0, 99.477, 98.5, 50.0, 0.0):
                mod = types.SimpleNamespace(K=K, R=R, activation_percentile=pct)
                r, dr, sk = v57.split_select_params(mod)
                scalars.append({"K": K, "ratio": ratio, "R": R, "pct": pct,
                                "descending_rank": int(dr), "select_k": int(sk)})
    (out / "scalars.json").write_text(json.dumps(scalars, indent=0))

    # ---- select + fake quant --------------------------------------------------------
    cases = [(8, 64, 0.05, 100.0, 1), (6, 256, 0.10, 100.0, 2), (4, 4096, 0.05, 100.0, 3),
             (4, 4096, 0.005, 98.5, 4), (3, 1024, 0.02, 99.477, 5)]
    blob = {}
    for ci, (M, K, ratio, pct, seed) in enumerate(cases):
        xb = distinct_rows(M, K, seed)
        A = torch.from_numpy(bits_to_f32(xb).copy())
        R, body_thr, tail_thr, idx = cmp_.compute_thresholds_and_indices(A, ratio, pct)
        idx2, body2, tail2 = v38.current_select(A, R, pct)
        assert torch.equal(idx, idx2) and torch.equal(body_thr, body2) and torch.equal(tail_thr, tail2)
        recon = cmp_.fake_quant_reconstruct(A, body_thr, tail_thr, idx, 1e-8)
        blob[f"c{ci}_x_bits"] = xb
        blob[f"c{ci}_meta"] = np.array([M, K, R], dtype=np.int64)
        blob[f"c{ci}_pct"] = np.array([pct], dtype=np.float64)
        blob[f"c{ci}_idx"] = idx.numpy().astype(np.int32)
        blob[f"c{ci}_body_thr"] = body_thr.numpy().astype(np.float32)
        blob[f"c{ci}_tail_thr"] = tail_thr.numpy().astype(np.float32)
        blob[f"c{ci}_recon"] = recon.numpy().astype(np.float32)
    blob["n_cases"] = np.array([len(cases)], dtype=np.int64)

    # ---- nibble decode ---------------------------------------------------------------
    packed = torch.arange(256, dtype=torch.uint8)
    blob["nibble_packed"] = packed.numpy()
    blob["nibble_decoded"] = cmp_.decode_signed_int4(packed, 1, 512).numpy().astype(np.int8)

    # ---- RTN weights -------------------------------------------------------------------
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((24, 256), dtype=np.float32) * np.float32(0.02))
    w_bits = ((w.view(np.uint32) + 0x7FFF + ((w.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    w_bits[3, :] = 0  # an all-zero output channel exercises the eps clamp
    W = torch.from_numpy(bits_to_f32(w_bits).copy())
    scale = v29.make_rtn_scale_cpu(W, 1e-8)
    rargs = types.SimpleNamespace(w_asym=False, scale_eps=1e-8,
                                  weight_scale_stat_fn=lambda a, _args: a.amax(dim=-1, keepdim=True))
    wq, exact_scale = rtn.rtn_quantize_with_scale(W, bits=4, groupsize=-1, args=rargs)
    assert torch.equal(scale, exact_scale)
    blob["rtn_w_bits"] = w_bits
    blob["rtn_scale"] = scale.numpy().astype(np.float32)
    blob["rtn_wq"] = wq.numpy().astype(np.float32)
    np.savez_compressed(out / "reference_vectors.npz", **blob)

    # ---- policy loader -----------------------------------------------------------------
    pol_path = Path(args.reference) / "policies" / "qwen3_8b_fixed_ratio0p05_policy_v1.json"
    pol = v29.load_policy(pol_path, False)
    keys = sorted(pol["modules"])
    sample = {k: pol["modules"][k] for k in keys[:7] + keys[-7:]}
    (out / "policy_loader.json").write_text(json.dumps(
        {"n_modules": len(keys), "sample": sample,
         "raw_first": json.loads(pol_path.read_text())["modules"][keys[0]]["ratio"]
         if "ratio" in json.loads(pol_path.read_text())["modules"][keys[0]] else None}, indent=0))
    print("golden vectors written to", out)


if __name__ == "__main__":
    main()
