"""Weight I/O in the reference's on-disk format: safetensors shards of the Qwen3.5-0.8B checkpoint.

Mirrors the loader contract of the reference (engine/loader.h:4-14,118-141; name rules
specification/02-tokenization-and-embedding.md:70-81; shapes and dtypes
specification/01-weights-and-shapes.md:12-120; the torch loader speccheck/specimpl.py:60-127):

* shards are resolved from `model.safetensors.index.json` if present, else every `*.safetensors`
  file of the directory;
* names are normalised `model.language_model.* -> lm.*`, `mtp.layers.0.* -> mtp.layer0.*`,
  other `mtp.* -> mtp.*`; `model.visual.*` is skipped; any other tensor is a loud failure, and so
  is a name collision, a missing tensor, a wrong shape or a wrong dtype;
* the tied head: `lm_head.weight` does not exist in the checkpoint and is registered as a second
  NAME of the embedding storage (one blob, two names);
* the 36 F32 tensors (`linear_attn.A_log`, `linear_attn.norm.weight`) are cast to bf16 at load, as
  the reference's torch implementation does with its default `keep_f32_scalars=False`
  (speccheck/specimpl.py:83-85) - the form every parity gate of this repository is measured in;
* optional verification hashes (SHA-256) the bytes that ended up resident against the bytes of the
  file, per tensor, which proves name map, file offset, dtype and tying together.

The file format itself (8-byte little-endian header length, JSON header of
name -> {dtype, shape, data_offsets}, then the raw little-endian tensor bytes) is read and written
here directly; no third-party reader is needed on the product path.
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass, field
from pathlib import Path

import torch

from . import weights as W

_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
           "I64": (torch.int64, 8), "I32": (torch.int32, 4), "U8": (torch.uint8, 1)}
_DTYPE_NAMES = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16",
                torch.int64: "I64", torch.int32: "I32", torch.uint8: "U8"}
F32_SUFFIXES = ("linear_attn.A_log", "linear_attn.norm.weight")
LOAD, SKIP_VISION, UNKNOWN = "load", "skip_vision", "unknown"


class CheckpointError(RuntimeError):
    """Any violation of the loader contract (unknown tensor, collision, shape, dtype, truncation)."""


def normalize_name(checkpoint_name: str):
    """(plan, engine_name): the reference's name classification (engine/loader.h:29-33)."""
    if checkpoint_name.startswith("model.visual."):
        return SKIP_VISION, ""
    if checkpoint_name.startswith("model.language_model."):
        return LOAD, "lm." + checkpoint_name[len("model.language_model."):]
    if checkpoint_name.startswith("mtp.layers.0."):
        return LOAD, "mtp.layer0." + checkpoint_name[len("mtp.layers.0."):]
    if checkpoint_name.startswith("mtp.") and not checkpoint_name.startswith("mtp.layers."):
        return LOAD, checkpoint_name
    return UNKNOWN, ""


def denormalize_name(engine_name: str) -> str:
    """Inverse of normalize_name for loadable tensors."""
    if engine_name.startswith("lm."):
        return "model.language_model." + engine_name[3:]
    if engine_name.startswith("mtp.layer0."):
        return "mtp.layers.0." + engine_name[len("mtp.layer0."):]
    return engine_name


# ------------------------------------------------------------------------------------------------
# the container format
# ------------------------------------------------------------------------------------------------
@dataclass
class Entry:
    name: str
    dtype: str
    shape: tuple
    begin: int          # absolute file offsets of the tensor's bytes
    end: int
    shard: str


def read_header(path) -> tuple[dict, int]:
    """name -> Entry for one shard, plus the offset at which tensor data starts."""
    path = str(path)
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise CheckpointError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise CheckpointError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        try:
            meta = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not JSON: {e}") from None
    base = 8 + n
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        dt, shape, (b, e) = m["dtype"], tuple(int(x) for x in m["shape"]), m["data_offsets"]
        if dt not in _DTYPES:
            raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {dt}")
        numel = 1
        for d in shape:
            numel *= d
        if e - b != numel * _DTYPES[dt][1]:
            raise CheckpointError(f"{path}: tensor {name} spans {e - b} bytes, shape {shape} {dt} needs {numel * _DTYPES[dt][1]}")
        if base + e > size:
            raise CheckpointError(f"{path}: tensor {name} ends at {base + e}, file has {size} bytes (truncated shard)")
        out[name] = Entry(name, dt, shape, base + b, base + e, path)
    return out, base


def write_shard(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write name -> CPU tensor as one safetensors shard (tensors in name order, 8-byte aligned header)."""
    header, off = {}, 0
    names = sorted(tensors)
    for name in names:
        t = tensors[name]
        if t.dtype not in _DTYPE_NAMES:
            raise CheckpointError(f"cannot store dtype {t.dtype} ({name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in names:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")


def resolve_shards(model_dir) -> list[str]:
    """Shard paths: the index file's weight_map if there is one, else every *.safetensors file."""
    d = Path(model_dir)
    if d.is_file():
        return [str(d)]
    idx = d / "model.safetensors.index.json"
    if idx.exists():
        wm = json.loads(idx.read_text())["weight_map"]
        shards = sorted({str(d / v) for v in wm.values()})
    else:
        shards = sorted(str(p) for p in d.glob("*.safetensors"))
    if not shards:
        raise CheckpointError(f"{model_dir}: no safetensors shard found")
    for s in shards:
        if not os.path.exists(s):
            raise CheckpointError(f"{s}: shard named by the index is missing")
    return shards


# ------------------------------------------------------------------------------------------------
# the weight store
# ------------------------------------------------------------------------------------------------
@dataclass
class Weight:
    """One engine-visible tensor (engine/loader.h:60-74)."""
    name: str                 # normalised name this entry is registered under
    storage_owner: str        # normalised name whose allocation backs `tensor`
    checkpoint_name: str      # original name in the shard ("" for an engine alias)
    shape: tuple
    file_dtype: str           # dtype in the shard ("BF16" / "F32")
    tensor: torch.Tensor      # resident tensor (bf16)

    @property
    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()

    def is_alias(self) -> bool:
        return self.storage_owner != self.name

    def shape_string(self) -> str:
        return "x".join(str(d) for d in self.shape)


@dataclass
class LoadStats:
    shard_paths: list = field(default_factory=list)
    header_bytes: int = 0
    uploaded_bytes: int = 0
    n_loaded: int = 0
    n_skipped_vision: int = 0
    parse_ms: float = 0.0
    read_ms: float = 0.0
    verify_ms: float = 0.0
    total_ms: float = 0.0
    device_verified: bool = False
    n_verified: int = 0
    verify_failures: list = field(default_factory=list)


def expected_spec(vocab: int | None, layers, mtp: bool) -> dict:
    """checkpoint name -> (file dtype, shape) the text path must contain (the spec's tables)."""
    spec = {}
    for name, (_, shape) in W.full_spec(vocab or W.VOCAB, layers, mtp).items():
        spec[name] = ("F32" if name.endswith(F32_SUFFIXES) else "BF16", tuple(shape))
    return spec


class WeightStore:
    """Name-indexed resident weights of the text path (engine/loader.h:118-165)."""

    def __init__(self):
        self._slots: dict[str, Weight] = {}
        self.ckpt_to_engine: list[tuple[str, str]] = []
        self.skipped_vision_count = 0
        self._allocations = 0
        self._resident_bytes = 0

    # ---- lookups ------------------------------------------------------------------------------
    def at(self, name: str) -> Weight:
        try:
            return self._slots[name]
        except KeyError:
            raise CheckpointError(f"no weight named {name!r}") from None

    def find(self, name: str):
        return self._slots.get(name)

    def lookup_count(self) -> int:            # names, aliases included
        return len(self._slots)

    def allocation_count(self) -> int:
        return self._allocations

    def resident_bytes(self) -> int:
        return self._resident_bytes

    def checkpoint_dict(self) -> dict:
        """checkpoint name -> resident tensor: what `Engine(params, ...)` and the oracle consume."""
        return {w.checkpoint_name: w.tensor for w in self._slots.values() if not w.is_alias()}

    # ---- loading ------------------------------------------------------------------------------
    @staticmethod
    def load(model_dir, device: str = "cpu", vocab: int | None = None, layers=None, mtp: bool = True,
             verify: bool = False):
        """Load the text path of a checkpoint directory (or single shard).  Returns (store, stats).

        `vocab=None` accepts whatever row count the embedding has (the real one is 248,320);
        `layers=None` expects all 24 layers.  Raises CheckpointError on any contract violation.
        """
        import time
        t_start = time.perf_counter()
        store, stats = WeightStore(), LoadStats()
        stats.shard_paths = resolve_shards(model_dir)
        entries: dict[str, Entry] = {}
        t0 = time.perf_counter()
        for shard in stats.shard_paths:
            found, base = read_header(shard)
            stats.header_bytes += base
            for name, e in found.items():
                if name in entries:
                    raise CheckpointError(f"tensor {name} appears in {entries[name].shard} and in {shard}")
                entries[name] = e
        stats.parse_ms = (time.perf_counter() - t0) * 1e3

        # classify every tensor: load, skip, or fail loudly
        plan: dict[str, str] = {}
        for name in sorted(entries):
            kind, eng = normalize_name(name)
            if kind == SKIP_VISION:
                store.skipped_vision_count += 1
                continue
            if kind == UNKNOWN:
                raise CheckpointError(f"tensor {name} is neither loaded nor explicitly skipped")
            if eng in plan.values():
                raise CheckpointError(f"two checkpoint tensors normalise to {eng}")
            plan[name] = eng
        stats.n_skipped_vision = store.skipped_vision_count

        spec = expected_spec(vocab, layers, mtp)
        if not mtp:
            extra_mtp = [n for n in plan if n.startswith("mtp.")]
            for n in extra_mtp:                     # a text-only load ignores the MTP block
                del plan[n]
        missing = sorted(set(spec) - set(plan))
        if missing:
            raise CheckpointError(f"{len(missing)} tensors of the text path are missing, first: {missing[0]}")
        extra = sorted(set(plan) - set(spec))
        if extra:
            raise CheckpointError(f"{len(extra)} tensors are outside the text path's tables, first: {extra[0]}")
        for name, (dt, shape) in spec.items():
            e = entries[name]
            if name == W.LM + "embed_tokens.weight" and vocab is None:
                shape = (e.shape[0], W.D_MODEL) if len(e.shape) == 2 else shape
            if e.shape != shape:
                raise CheckpointError(f"{name}: shape {e.shape}, the text path needs {shape}")
            if e.dtype != dt:
                raise CheckpointError(f"{name}: dtype {e.dtype}, the checkpoint format has {dt}")

        # read (memory-mapped), cast the F32 scalars, move to the device
        t0 = time.perf_counter()
        maps = {}
        try:
            for shard in stats.shard_paths:
                f = open(shard, "rb")
                maps[shard] = (f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
            for name in sorted(plan):
                e = entries[name]
                mm = maps[e.shard][1]
                tdt = _DTYPES[e.dtype][0]
                if e.end > e.begin:
                    with warnings.catch_warnings():       # the map is read-only and only ever read
                        warnings.simplefilter("ignore", UserWarning)
                        raw = torch.frombuffer(mm, dtype=tdt, count=(e.end - e.begin) // _DTYPES[e.dtype][1], offset=e.begin)
                    t = raw.reshape(e.shape).to(torch.bfloat16).clone() if device == "cpu" else \
                        raw.reshape(e.shape).to(device).to(torch.bfloat16)
                else:
                    t = torch.empty(e.shape, dtype=torch.bfloat16, device=device)
                eng = plan[name]
                store._slots[eng] = Weight(eng, eng, name, e.shape, e.dtype, t)
                store.ckpt_to_engine.append((name, eng))
                store._allocations += 1
                store._resident_bytes += t.numel() * t.element_size()
            stats.read_ms = (time.perf_counter() - t0) * 1e3

            # the tied head: a second name for the embedding's storage, no second copy
            emb = store._slots["lm.embed_tokens.weight"]
            if "lm_head.weight" in store._slots:
                raise CheckpointError("lm_head.weight exists in a checkpoint that ties the head to the embedding")
            store._slots["lm_head.weight"] = Weight("lm_head.weight", emb.name, "", emb.shape, emb.file_dtype, emb.tensor)
            stats.n_loaded = len(plan)
            stats.uploaded_bytes = store._resident_bytes

            if verify:
                t0 = time.perf_counter()
                for name in sorted(plan):
                    e = entries[name]
                    w = store._slots[plan[name]]
                    mm = maps[e.shard][1]
                    if e.dtype == "BF16":
                        want = hashlib.sha256(mm[e.begin:e.end]).hexdigest()
                    else:       # resident form of an F32 scalar is its bf16 rounding
                        with warnings.catch_warnings():
                            warnings.simplefilter("ignore", UserWarning)
                            src = torch.frombuffer(mm, dtype=torch.float32, count=(e.end - e.begin) // 4, offset=e.begin)
                        want = hashlib.sha256(src.to(torch.bfloat16).view(torch.uint8).numpy().tobytes()).hexdigest()
                    got = hashlib.sha256(w.tensor.detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()).hexdigest()
                    stats.n_verified += 1
                    if got != want:
                        stats.verify_failures.append(f"{name}: resident bytes differ from the shard")
                head = store._slots["lm_head.weight"].tensor
                if head.data_ptr() != emb.tensor.data_ptr():
                    stats.verify_failures.append("lm_head.weight is not the embedding's storage")
                stats.device_verified = not stats.verify_failures
                stats.verify_ms = (time.perf_counter() - t0) * 1e3
        finally:
            for f, mm in maps.values():
                try:
                    mm.close()
                except BufferError:
                    pass                      # a CPU tensor still views the map; it is released with it
                f.close()
        store.ckpt_to_engine.sort()
        stats.total_ms = (time.perf_counter() - t_start) * 1e3 - stats.verify_ms
        return store, stats


def save_checkpoint(params: dict, model_dir, n_vision_dummies: int = 0, shard_name: str = "model.safetensors-00001-of-00001.safetensors",
                    write_index: bool = False) -> str:
    """Write checkpoint-named tensors as a one-shard checkpoint directory in the reference's
    format: A_log / gated-norm weights as F32, everything else BF16, plus (for tests of the skip
    rule) `n_vision_dummies` tiny `model.visual.*` tensors."""
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    out = {}
    for name, t in params.items():
        t = t.detach().cpu()
        out[name] = t.to(torch.float32) if name.endswith(F32_SUFFIXES) else t.to(torch.bfloat16)
    for i in range(n_vision_dummies):
        out[f"model.visual.blocks.{i}.dummy.weight"] = torch.zeros(4, dtype=torch.bfloat16)
    path = d / shard_name
    write_shard(path, out, {"format": "pt"})
    if write_index:
        (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": {n: shard_name for n in out}}))
    return str(path)
