"""On-disk format of a prepared weight, so that a model loads without rotating and re-quantising.

The reference re-quantises every linear at start-up (tools/bench_multimodel_all_layers_policy_fastqf_v29.py:
`prepare_layer`); it has no such file.  Layout of a `.tqw` file (little endian):

    bytes 0..7    magic  b"TQW1\\0\\0\\0\\0"
    bytes 8..15   u64    length H of the JSON header
    bytes 16..    H bytes of UTF-8 JSON:
                  {"N", "K", "had_kind", "eps", "ratio", "activation_percentile", "policy_hash",
                   "epilogue", "rms_eps",
                   "tensors": {name: {"dtype", "shape", "offset", "nbytes", "crc32"}}}
    then the tensor payloads, each starting at its `offset` (from the start of the file, 256-byte aligned),
    raw row-major bytes.

Stored tensors: `b_col` u8 [N, K/2] (packed INT4 codes, element 2i in the low nibble), `w_scale` f32 [N],
and when present `w_rot` bf16 [N, K] (rotated weights, the tail operand), `b_row` u8 [K, N/2], `bias` f32 [N],
`rms_weight` bf16 [K] (the RMSNorm a layer applies inside its prologue; `epilogue` names its fused activation).
`w_t` ([K, N], the transpose of `w_rot`) is not stored: the loader rebuilds it when asked for.
"""
from __future__ import annotations

import hashlib
import json
import struct
import zlib
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from .ops import PreparedWeight

MAGIC = b"TQW1\0\0\0\0"
_ALIGN = 256
_DTYPES = {"uint8": torch.uint8, "float32": torch.float32, "bfloat16": torch.bfloat16}


def policy_hash(entry: Optional[dict]) -> str:
    """Short stable hash of a policy entry (ratio, percentiles), stored so that a stale file is noticed."""
    if not entry:
        return ""
    blob = json.dumps({k: entry[k] for k in sorted(entry)}, sort_keys=True).encode()
    return hashlib.sha256(blob).hexdigest()[:16]


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        t = t.view(torch.int16)
    return t.numpy().tobytes()


def save_prepared(path, w: PreparedWeight, ratio: Optional[float] = None, activation_percentile: float = 100.0,
                  policy_entry: Optional[dict] = None, eps: Optional[float] = None, epilogue: str = "none",
                  rms_weight: Optional[torch.Tensor] = None, rms_eps: float = 1e-6) -> None:
    tensors = {"b_col": w.b_col, "w_scale": w.w_scale}
    if rms_weight is not None:
        tensors["rms_weight"] = rms_weight
    w_rot = w.w_rot if w.w_rot is not None else (w.w_t.t().contiguous() if w.w_t is not None else None)
    if w_rot is not None:
        tensors["w_rot"] = w_rot
    if w.b_row is not None:
        tensors["b_row"] = w.b_row
    if w.bias is not None:
        tensors["bias"] = w.bias
    payloads = {k: _raw_bytes(v) for k, v in tensors.items()}
    header = {"N": int(w.N), "K": int(w.K), "had_kind": int(w.had_kind), "eps": eps, "ratio": ratio,
              "activation_percentile": activation_percentile, "policy_hash": policy_hash(policy_entry), "epilogue": epilogue,
              "rms_eps": float(rms_eps), "tensors": {}}
    # the header's own length moves the offsets: lay it out with offsets as fixed-width numbers first
    for k, v in tensors.items():
        header["tensors"][k] = {"dtype": str(v.dtype).replace("torch.", ""), "shape": list(v.shape),
                                "offset": 0, "nbytes": len(payloads[k]), "crc32": zlib.crc32(payloads[k]) & 0xffffffff}
    probe = json.dumps(header).encode()
    pos = (16 + len(probe) + 64 * len(tensors) + _ALIGN - 1) // _ALIGN * _ALIGN  # room for the real offsets
    for k in tensors:
        header["tensors"][k]["offset"] = pos
        pos = (pos + len(payloads[k]) + _ALIGN - 1) // _ALIGN * _ALIGN
    hjson = json.dumps(header).encode()
    first = min(t["offset"] for t in header["tensors"].values())
    if 16 + len(hjson) > first:
        raise RuntimeError("prepared-weight header does not fit before the first tensor")
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for k in tensors:
            f.seek(header["tensors"][k]["offset"])
            f.write(payloads[k])
        f.truncate(pos)


def read_header(path) -> dict:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise RuntimeError(f"{path}: not a prepared-weight file (bad magic)")
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen > 1 << 20:
            raise RuntimeError(f"{path}: implausible header length {hlen}")
        return json.loads(f.read(hlen).decode())


def _read_tensor(f, path, name: str, d: dict, size: int, verify: bool, device) -> torch.Tensor:
    if d["dtype"] not in _DTYPES:
        raise RuntimeError(f"{path}: tensor {name} has unknown dtype {d['dtype']}")
    if d["offset"] % _ALIGN or d["offset"] + d["nbytes"] > size:
        raise RuntimeError(f"{path}: tensor {name} lies outside the file")
    f.seek(d["offset"])
    raw = f.read(d["nbytes"])
    if len(raw) != d["nbytes"]:
        raise RuntimeError(f"{path}: tensor {name} is truncated")
    if verify and (zlib.crc32(raw) & 0xffffffff) != d["crc32"]:
        raise RuntimeError(f"{path}: tensor {name} fails its checksum")
    dt = _DTYPES[d["dtype"]]
    np_dt = {torch.uint8: np.uint8, torch.float32: np.float32, torch.bfloat16: np.int16}[dt]
    arr = np.frombuffer(raw, dtype=np_dt).reshape(d["shape"]).copy()
    t = torch.from_numpy(arr)
    if dt == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.to(device)


def load_extra(path, name: str, device="cuda", verify: bool = True) -> Optional[torch.Tensor]:
    """One named tensor of a `.tqw` file (e.g. "rms_weight"), or None when the file does not hold it."""
    path = Path(path)
    d = read_header(path)["tensors"].get(name)
    if d is None:
        return None
    with open(path, "rb") as f:
        return _read_tensor(f, path, name, d, path.stat().st_size, verify, device)


def load_prepared(path, device="cuda", need_w_t: bool = False, keep_w_rot: bool = True, verify: bool = True,
                  expect_policy_entry: Optional[dict] = None) -> PreparedWeight:
    """Reads a `.tqw` file onto `device`.  `need_w_t` rebuilds the [K, N] transpose (gather engine and decode tail);
    `verify` checks the CRC of every tensor; `expect_policy_entry` refuses a file written for another policy."""
    path = Path(path)
    h = read_header(path)
    if expect_policy_entry is not None and h.get("policy_hash") != policy_hash(expect_policy_entry):
        raise RuntimeError(f"{path}: written for another policy entry")
    size = path.stat().st_size
    out = {}
    with open(path, "rb") as f:
        for name, d in h["tensors"].items():
            out[name] = _read_tensor(f, path, name, d, size, verify, device)
    N, K = int(h["N"]), int(h["K"])
    if tuple(out["b_col"].shape) != (N, K // 2) or tuple(out["w_scale"].shape) != (N,):
        raise RuntimeError(f"{path}: tensor shapes disagree with N = {N}, K = {K}")
    w_rot = out.get("w_rot")
    w_t = w_rot.t().contiguous() if (need_w_t and w_rot is not None) else None
    return PreparedWeight(N, K, int(h["had_kind"]), out["b_col"], out["w_scale"], w_t, out.get("b_row"),
                          w_rot if keep_w_rot else None, out.get("bias"))
