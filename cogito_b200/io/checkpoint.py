"""COG1 checkpoints: byte-compatible with cg_save_model / cg_load_model
(include/cg_serialization.h:11-31, src/core/serialization.c:9-77).

Layout (little-endian): 24-byte header {magic 0x434F4731, version, num_tensors, pad,
total_size}; ``num_tensors`` directory entries of 120 bytes {name[64], ndim i32, shape[8] i32,
dtype i32, offset u64, size_bytes u64}; then the payloads back to back.  The reference writes
fp32 only (dtype 0) and leaves total_size 0; this writer also fills total_size and uses
dtype 1 for bf16 payloads and dtype 2 for packed INT4 payloads (each followed by a
``<name>.scales`` fp32 entry; ``cg_load_model`` dequantises such a pair into one fp32 tensor).
Tensors of other types (integer counters, bool masks, fp64, fp16) keep their exact bytes under
type codes of this library (16 and up), which a reader of the reference's format does not know.

On top of the tensor file: a ``*.state`` sidecar (same format) with the optimizer moments, fp32
master weights, step counters, loss-scale state and RNG seeds, so that a resumed run
continues bit-for-bit; and per-rank shard files named by (dp, tp, pp) coordinates.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch

MAGIC = 0x434F4731
HEADER = struct.Struct("<IIIIQ")                     # magic, version, count, pad, total_size
ENTRY = struct.Struct("<64si8iiQQ")                  # name, ndim, shape[8], dtype, offset, size
DT_FP32, DT_BF16, DT_INT4 = 0, 1, 2
# exact-byte payloads of this library (not part of the reference's enum)
RAW_CODES = {torch.int64: 16, torch.int32: 17, torch.uint8: 18, torch.bool: 19, torch.float64: 20,
             torch.float16: 21, torch.int16: 22, torch.int8: 23}
RAW_NUMPY = {16: np.int64, 17: np.int32, 18: np.uint8, 19: np.bool_, 20: np.float64, 21: np.float16,
             22: np.int16, 23: np.int8}
assert HEADER.size == 24 and ENTRY.size == 120


def _payload(t: torch.Tensor, int4: bool):
    t = t.detach().cpu().contiguous()
    if int4:
        if t.dtype != torch.uint8:
            raise TypeError("a packed INT4 payload must be a uint8 tensor")
        return DT_INT4, t.numpy().tobytes()
    if t.dtype == torch.bfloat16:
        return DT_BF16, t.view(torch.int16).numpy().tobytes()
    if t.dtype == torch.float32:
        return DT_FP32, t.numpy().tobytes()
    if t.dtype in RAW_CODES:
        return RAW_CODES[t.dtype], t.numpy().tobytes()
    raise TypeError(f"cannot store a tensor of type {t.dtype} in a COG1 file")


def save_tensors(path: str, tensors: dict[str, torch.Tensor], int4_shapes: dict[str, tuple] | None = None) -> int:
    """Write a COG1 file.  The uint8 tensors named in ``int4_shapes`` are packed INT4 payloads whose
    logical shape is ``int4_shapes[name]``; every other tensor keeps its type.  Returns the number
    of bytes written."""
    names = list(tensors)
    entries, blobs = [], []
    off = HEADER.size + ENTRY.size * len(names)
    for name in names:
        raw = name.encode()
        if len(raw) > 63:
            raise ValueError(f"tensor name longer than 63 bytes: {name}")
        t = tensors[name]
        is_int4 = bool(int4_shapes) and name in int4_shapes
        dtype, blob = _payload(t, is_int4)
        shape = tuple(int4_shapes[name]) if is_int4 else tuple(t.shape)
        if len(shape) > 8:
            raise ValueError("at most 8 dimensions")
        entries.append(ENTRY.pack(raw, len(shape), *(list(shape) + [0] * (8 - len(shape))), dtype, off, len(blob)))
        blobs.append(blob)
        off += len(blob)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(HEADER.pack(MAGIC, 1, len(names), 0, off))
        for e in entries:
            f.write(e)
        for b in blobs:
            f.write(b)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)                            # a crash never leaves a half-written checkpoint
    return off


def load_tensors(path: str, device="cpu", use_mmap: bool = True) -> dict[str, torch.Tensor]:
    """Read a COG1 file (also files written by the reference: fp32 payloads, total_size 0)."""
    with open(path, "rb") as f:
        buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if use_mmap else f.read()
    if len(buf) < HEADER.size:
        raise ValueError("not a COG1 file: too short")
    magic, version, count, _pad, _total = HEADER.unpack_from(buf, 0)
    if magic != MAGIC:
        raise ValueError(f"not a COG1 file: magic {magic:#x}")
    out = {}
    for i in range(count):
        raw, ndim, *rest = ENTRY.unpack_from(buf, HEADER.size + i * ENTRY.size)
        shape, dtype, offset, size = rest[:8][:ndim], rest[8], rest[9], rest[10]
        name = raw.split(b"\0", 1)[0].decode()
        if offset + size > len(buf):
            raise ValueError(f"entry {name} points past the end of the file")
        shape = tuple(shape)
        if dtype == DT_FP32:
            t = torch.from_numpy(np.frombuffer(buf, np.float32, size // 4, offset).copy()).reshape(shape)
        elif dtype == DT_BF16:
            t = torch.from_numpy(np.frombuffer(buf, np.int16, size // 2, offset).copy()).view(torch.bfloat16).reshape(shape)
        elif dtype == DT_INT4:
            t = torch.from_numpy(np.frombuffer(buf, np.uint8, size, offset).copy())
            t.logical_shape = shape
        elif dtype in RAW_NUMPY:
            npdt = np.dtype(RAW_NUMPY[dtype])
            t = torch.from_numpy(np.frombuffer(buf, npdt, size // npdt.itemsize, offset).copy()).reshape(shape)
        else:
            raise ValueError(f"entry {name}: unknown dtype {dtype}")
        out[name] = t.to(device)
    return out


def shard_path(base: str, dp: int, tp: int, pp: int) -> str:
    return f"{base}.dp{dp:02d}.tp{tp:02d}.pp{pp:02d}.cog"


def save_model(path: str, model: torch.nn.Module) -> int:
    return save_tensors(path, {k: v for k, v in model.state_dict().items()})


def load_model(path: str, model: torch.nn.Module, strict: bool = True) -> None:
    state = load_tensors(path)
    own = model.state_dict()
    missing = [k for k in own if k not in state]
    if strict and missing:
        raise KeyError(f"checkpoint lacks {missing[:5]}")
    with torch.no_grad():
        for k, v in own.items():
            if k in state:
                v.copy_(state[k].to(v.device, v.dtype).view_as(v))


# ---------------------------------------------------------------- training state
def save_training_state(base: str, model, opt, step: int, extra: dict | None = None) -> None:
    """``base``.cog: parameters; ``base``.state: optimizer tensors + a JSON blob (as a uint8-free
    fp32-coded entry) with counters, loss-scale state and seeds."""
    save_model(base + ".cog", model)
    tensors = {f"opt.{k}": v for k, v in opt.state_tensors().items()}
    scaler = opt.scaler.state_dict() if getattr(opt, "scaler", None) is not None else {}
    meta = {"step": int(step), "lr": float(opt.lr), "scaler": scaler, "extra": extra or {},
            "torch_rng": torch.get_rng_state().tolist()}
    blob = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8).astype(np.float32)
    tensors["meta.json"] = torch.from_numpy(blob)
    save_tensors(base + ".state", tensors)


def load_training_state(base: str, model, opt) -> dict:
    load_model(base + ".cog", model)
    state = load_tensors(base + ".state")
    meta = json.loads(bytes(state.pop("meta.json").to(torch.uint8).tolist()).decode())
    own = opt.state_tensors()
    with torch.no_grad():
        for k, v in own.items():
            v.copy_(state[f"opt.{k}"].to(v.device, v.dtype).view_as(v))
    if "master" not in own and hasattr(opt, "refresh_master"):
        opt.refresh_master()
    opt.lr = meta["lr"]
    if meta["scaler"] and getattr(opt, "scaler", None) is not None:
        opt.scaler.load_state_dict(meta["scaler"])
    torch.set_rng_state(torch.tensor(meta["torch_rng"], dtype=torch.uint8))
    return meta


def dp_shard_path(base: str, rank: int, ranks: int) -> str:
    return f"{base}.opt.dp{rank:02d}of{ranks:02d}.state"


def save_dp_optimizer_shard(base: str, opt) -> str:
    """Write this data-parallel rank's optimizer shard (``DPFusedAdam.shard_state``): Adam moments,
    fp32 master weights, the parts of the flat vector they belong to, step and loss-scale state."""
    sh = opt.shard_state()
    tensors = {k: sh[k] for k in ("m", "v", "master") if sh.get(k) is not None}
    meta = {k: sh[k] for k in ("segments", "n", "ranks")}
    meta["scaler"] = sh["scaler"]
    tensors["meta.json"] = torch.from_numpy(np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8).astype(np.float32))
    path = dp_shard_path(base, opt.rank, opt.ranks)
    save_tensors(path, tensors)
    return path


def load_dp_optimizer_resharded(base: str, opt) -> int:
    """Restore ``opt`` (a ``DPFusedAdam`` of the CURRENT group, whatever its size) from the shard
    files a previous run wrote under ``base``; returns the data-parallel size of that run.  The
    parameters must have been loaded before (``load_model``)."""
    import glob
    import re
    files = sorted(glob.glob(glob.escape(base) + ".opt.dp*of*.state"))
    if not files:
        raise FileNotFoundError(f"no optimizer shards under {base}")
    old = {int(re.search(r"of(\d+)\.state$", f).group(1)) for f in files}
    if len(old) != 1 or len(files) != next(iter(old)):
        raise ValueError(f"incomplete or mixed shard set under {base}: {files}")
    shards = []
    for f in files:
        state = load_tensors(f)
        meta = json.loads(bytes(state.pop("meta.json").to(torch.uint8).tolist()).decode())
        meta.update(state)
        shards.append(meta)
    opt.load_resharded(shards)
    return next(iter(old))


def gather_shards(base: str, dp: int, tp: int, pp: int) -> dict[str, torch.Tensor]:
    """Read every (tp, pp) shard of data-parallel replica 0 into one name -> tensor map with the
    coordinates prefixed (``tp0.pp1.<name>``); a model-specific merge turns it into full weights."""
    out = {}
    for p in range(pp):
        for t in range(tp):
            for k, v in load_tensors(shard_path(base, 0, t, p)).items():
                out[f"tp{t}.pp{p}.{k}"] = v
    return out
