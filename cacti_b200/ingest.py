"""Checkpoint ingest: safetensors and torch-pickle directories -> device buffers of the training step.

Mirrors the reference's readers for the data that feeds the hot path:
  * `TensorsDir`  - src/util/safetensor.rs:30-145: `model.safetensors`, else the sorted `model-*-of-*.safetensors`
                    shards; header parsed without touching tensor bytes; duplicate names across shards are an error;
                    `get(key)` returns the type and a memory-mapped byte range (files are mapped lazily, once).
  * `PickleDir`   - src/util/safepickle.rs:36-197: `pytorch_model.bin`, else `pytorch_model-*-of-*.bin`; the pickle
                    stream is *interpreted, never executed*: only the handful of globals a state dict needs are
                    recognised and they build inert records; tensors must be packed (contiguous) and their bytes are
                    memory-mapped straight out of the zip archive (stored entries, 64-byte aligned as torch writes them).
  * `CellMatcher` - src/util/cell.rs match_: a pattern is a tuple of ints and strings consumed left to right against
                    the '.'-separated tokens of a key (an int must equal a token, a string may be a substring of one);
                    the first key in sorted order that consumes the whole pattern is taken and removed.
  * `match_llama` - src/librarium/llama.rs:284-303: the patterns of the decoder's parameters.
  * `load_llama`  - what examples/open_llama_3b_train.rs:203-260 does with `mem_set_yield_`: every matched tensor is
                    copied into its device buffer.  Here the bytes go mmap -> pinned staging ring -> async H2D on a copy
                    stream, so the page-cache reads of tensor i+1 overlap the transfer of tensor i.
"""
from __future__ import annotations

import glob
import io
import json
import mmap
import os
import pickle
import struct
import zipfile
from dataclasses import dataclass

import numpy as np

# safetensors dtype tag -> (numpy dtype or None, bytes per element); bf16 has no numpy type and is carried as uint16
ST_DTYPES = {"F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (None, 2),
             "I64": (np.int64, 8), "I32": (np.int32, 4), "I16": (np.int16, 2), "I8": (np.int8, 1), "U8": (np.uint8, 1),
             "BOOL": (np.bool_, 1)}
# torch storage class name -> safetensors-style tag
TORCH_STORAGE = {"DoubleStorage": "F64", "FloatStorage": "F32", "HalfStorage": "F16", "BFloat16Storage": "BF16",
                 "LongStorage": "I64", "IntStorage": "I32", "ShortStorage": "I16", "CharStorage": "I8",
                 "ByteStorage": "U8", "BoolStorage": "BOOL"}


class IngestError(Exception):
    """kind is one of the reference's error variants: Path, File, TensorsDict, PickleFile, DuplicateName."""

    def __init__(self, kind, detail=""):
        super().__init__(f"{kind}: {detail}" if detail else kind)
        self.kind = kind


@dataclass
class TensorEntry:
    dtype: str            # safetensors-style tag
    shape: tuple
    off: int              # byte range inside the file
    eoff: int

    @property
    def span_bytes(self):
        n = 1
        for d in self.shape:
            n *= d
        return n * ST_DTYPES[self.dtype][1]


class _Dir:
    """Shared part of the two readers: name -> (file index, entry), lazily mapped files."""

    def __init__(self, dir_path):
        self.dir_path = str(dir_path)
        self.model_paths, self.serial_key, self.tensor_map, self._maps = [], [], {}, []

    def _pick_files(self, single, pattern):
        p = os.path.join(self.dir_path, single)
        if os.path.isfile(p):
            return [p]
        files = sorted(glob.glob(os.path.join(self.dir_path, pattern)))
        if not files:
            raise IngestError("Path", f"no {single} or {pattern} in {self.dir_path}")
        return files

    def _add(self, name, entry):
        if name in self.tensor_map:
            raise IngestError("DuplicateName", name)
        self.serial_key.append(name)
        self.tensor_map[name] = (len(self.model_paths) - 1, entry)

    def clone_keys(self):
        return set(self.tensor_map)

    def get(self, key):
        """(dtype tag, shape, memoryview of the packed bytes).  An unknown key is a bug of the caller (the reference panics)."""
        idx, e = self.tensor_map[key]
        if e.span_bytes != e.eoff - e.off:
            raise IngestError("TensorsDict", f"{key}: {e.span_bytes} bytes by shape, {e.eoff - e.off} in file")
        if self._maps[idx] is None:
            with open(self.model_paths[idx], "rb") as f:
                self._maps[idx] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return e.dtype, e.shape, memoryview(self._maps[idx])[e.off:e.eoff]

    def close(self):
        for i, m in enumerate(self._maps):
            if m is not None:
                try:
                    m.close()
                except BufferError:          # a caller still holds a view; the map goes with the last view
                    pass
                self._maps[i] = None


class TensorsDir(_Dir):
    @classmethod
    def open(cls, dir_path):
        self = cls(dir_path)
        for path in self._pick_files("model.safetensors", "model-*-of-*.safetensors"):
            try:
                f = open(path, "rb")
            except OSError as e:
                raise IngestError("File", str(e))
            with f:
                size = os.fstat(f.fileno()).st_size
                head = f.read(8)
                if len(head) != 8:
                    raise IngestError("TensorsDict", f"{path}: truncated length prefix")
                (hlen,) = struct.unpack("<Q", head)
                if hlen > size - 8 or hlen > (100 << 20):
                    raise IngestError("TensorsDict", f"{path}: header length {hlen} out of range")
                try:
                    header = json.loads(f.read(hlen).decode("utf-8"))
                except (UnicodeDecodeError, json.JSONDecodeError) as e:
                    raise IngestError("TensorsDict", f"{path}: {e}")
            if not isinstance(header, dict):
                raise IngestError("TensorsDict", f"{path}: header is not an object")
            self.model_paths.append(path)
            self._maps.append(None)
            buf_start = 8 + hlen
            for name, ent in header.items():
                if name == "__metadata__":
                    continue
                try:
                    dtype, shape, (o0, o1) = ent["dtype"], tuple(int(d) for d in ent["shape"]), ent["data_offsets"]
                except (KeyError, TypeError, ValueError) as e:
                    raise IngestError("TensorsDict", f"{path}: entry {name}: {e}")
                if dtype not in ST_DTYPES or any(d < 0 for d in shape) or not (0 <= o0 <= o1 <= size - buf_start):
                    raise IngestError("TensorsDict", f"{path}: entry {name}: bad dtype, shape or offsets")
                self._add(name, TensorEntry(dtype, shape, buf_start + o0, buf_start + o1))
        return self


# ---- torch pickle, interpreted ----------------------------------------------------------------------------------
@dataclass
class _StorageRef:
    dtype: str
    key: str
    numel: int


@dataclass
class _TensorRec:
    storage: _StorageRef
    storage_offset: int
    shape: tuple
    stride: tuple


class _StorageType:
    def __init__(self, tag):
        self.tag = tag


def _rebuild_tensor_v2(storage, storage_offset, size, stride, *unused):
    # every value here comes from the file: check the types and signs before anything is computed from them
    if not isinstance(storage, _StorageRef) or not isinstance(storage_offset, int) or isinstance(storage_offset, bool):
        raise IngestError("PickleFile", "tensor record does not refer to a storage")
    if not isinstance(size, (tuple, list)) or not isinstance(stride, (tuple, list)):
        raise IngestError("PickleFile", "tensor record without a shape")
    if any(not isinstance(d, int) or isinstance(d, bool) or d < 0 for d in tuple(size) + tuple(stride)) or storage_offset < 0:
        raise IngestError("PickleFile", "negative or non-integer offset, dimension or stride")
    return _TensorRec(storage, int(storage_offset), tuple(size), tuple(stride))


def _rebuild_parameter(data, *unused):
    return data


class _InertUnpickler(pickle.Unpickler):
    """Builds records only.  Any global outside the list below ends the parse: nothing from the file is ever called."""

    def find_class(self, module, name):
        if module == "collections" and name == "OrderedDict":
            return dict
        if module == "torch._utils" and name == "_rebuild_tensor_v2":
            return _rebuild_tensor_v2
        if module == "torch._utils" and name == "_rebuild_parameter":
            return _rebuild_parameter
        if module == "torch" and name in TORCH_STORAGE:
            return _StorageType(TORCH_STORAGE[name])
        raise IngestError("PickleFile", f"global {module}.{name} is not part of a tensor state dict")

    def persistent_load(self, pid):
        if not (isinstance(pid, tuple) and len(pid) >= 5 and pid[0] == "storage" and isinstance(pid[1], _StorageType)):
            raise IngestError("PickleFile", "unexpected persistent id")
        if not isinstance(pid[4], int) or isinstance(pid[4], bool) or pid[4] < 0 or not isinstance(pid[2], (str, int)):
            raise IngestError("PickleFile", "malformed storage record")
        return _StorageRef(pid[1].tag, str(pid[2]), int(pid[4]))


def _stored_entry_offset(f, info):
    """File offset of the bytes of a stored (uncompressed) zip entry."""
    if info.compress_type != zipfile.ZIP_STORED:
        raise IngestError("PickleFile", f"{info.filename} is compressed; tensors must be stored entries")
    f.seek(info.header_offset)
    lh = f.read(30)
    if len(lh) != 30 or lh[:4] != b"PK\x03\x04":
        raise IngestError("PickleFile", f"{info.filename}: bad local header")
    nlen, xlen = struct.unpack("<HH", lh[26:30])
    return info.header_offset + 30 + nlen + xlen


class PickleDir(_Dir):
    @classmethod
    def open(cls, dir_path, prefix="pytorch_model"):
        self = cls(dir_path)
        self.prefix = prefix
        for path in self._pick_files(f"{prefix}.bin", f"{prefix}-*-of-*.bin"):
            try:
                zf = zipfile.ZipFile(path)
            except (OSError, zipfile.BadZipFile) as e:
                raise IngestError("PickleFile", f"{path}: {e}")
            with zf, open(path, "rb") as raw:
                names = zf.namelist()
                pkl = [n for n in names if n.endswith("/data.pkl") or n == "data.pkl"]
                if len(pkl) != 1:
                    raise IngestError("PickleFile", f"{path}: expected one data.pkl, found {len(pkl)}")
                root = pkl[0][: -len("data.pkl")]
                try:
                    state = _InertUnpickler(io.BytesIO(zf.read(pkl[0]))).load()
                except IngestError:
                    raise
                except Exception as e:            # malformed stream
                    raise IngestError("PickleFile", f"{path}: {type(e).__name__}: {e}")
                if not isinstance(state, dict):
                    raise IngestError("PickleFile", f"{path}: the pickled object is not a state dict")
                self.model_paths.append(path)
                self._maps.append(None)
                infos = {i.filename: i for i in zf.infolist()}
                for name, t in state.items():
                    if not isinstance(t, _TensorRec):
                        continue
                    info = infos.get(f"{root}data/{t.storage.key}")
                    if info is None:
                        raise IngestError("PickleFile", f"{path}: storage {t.storage.key} of {name} is missing")
                    if t.storage.dtype not in ST_DTYPES:
                        raise IngestError("PickleFile", f"{name}: unsupported storage type {t.storage.dtype}")
                    esz = ST_DTYPES[t.storage.dtype][1]
                    # packed layout only (src/util/safepickle.rs:147-156)
                    packed, acc = [], 1
                    for d in reversed(t.shape):
                        packed.append(acc)
                        acc *= d
                    if tuple(reversed(packed)) != t.stride[len(t.stride) - len(t.shape):]:
                        raise IngestError("PickleFile", f"{name}: strided (non-packed) tensors are not supported")
                    base = _stored_entry_offset(raw, info)
                    off = base + t.storage_offset * esz
                    eoff = off + acc * esz
                    if not (base <= off <= eoff <= base + info.file_size) or t.storage.numel * esz != info.file_size:
                        raise IngestError("PickleFile", f"{name}: tensor does not fit its storage")
                    if base % 64:
                        raise IngestError("PickleFile", f"{name}: storage is not 64-byte aligned in the archive")
                    self._add(str(name), TensorEntry(t.storage.dtype, t.shape, off, eoff))
        return self


# ---- matching ------------------------------------------------------------------------------------------------------
class CellMatcher:
    def __init__(self):
        self.rule = []

    def insert(self, pattern, target):
        self.rule.append((pattern if isinstance(pattern, tuple) else (pattern,), target))

    def match_(self, keys):
        """[(key, target)] for the patterns that found a key, in rule order; each key is used once."""
        keys = sorted(keys)
        out = []
        for pat, target in self.rule:
            for key in keys:
                idx = 0
                for tok in key.split("."):
                    want = pat[idx]
                    if (tok == str(want)) if isinstance(want, int) else (want in tok):
                        idx += 1
                        if idx == len(pat):
                            break
                if idx == len(pat):
                    keys.remove(key)
                    out.append((key, target))
                    break
        return out


def match_llama(n_layers, keys):
    """{parameter path: checkpoint key}; parameter paths are 'embed', 'lm_head', 'head_norm', 'layers.<i>.<name>'."""
    m = CellMatcher()
    m.insert("embed", "embed")
    for i in range(n_layers):
        m.insert((i, "input_layernorm"), f"layers.{i}.pre_norm")
        for ours, theirs in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "o_proj")):
            m.insert((i, "attn", theirs), f"layers.{i}.{ours}")
        m.insert((i, "post_attention_layernorm"), f"layers.{i}.post_norm")
        for ours in ("gate", "up", "down"):
            m.insert((i, "mlp", ours), f"layers.{i}.{ours}")
    m.insert("norm", "head_norm")
    m.insert("lm_head", "lm_head")
    return {target: key for key, target in m.match_(keys)}


# ---- mmap -> pinned staging -> device ------------------------------------------------------------------------------
def _torch_dtype(tag):
    import torch
    return {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64,
            "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}[tag]


def _as_u8(torch, view):
    """A uint8 tensor over a read-only byte range (it is only ever read)."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        return torch.frombuffer(view, dtype=torch.uint8)


class StagedCopier:
    """Copies byte ranges into device tensors through a ring of pinned buffers on its own stream.  `flush()` waits for
    everything issued.  On a CPU destination it copies directly (used by the tests that run without a GPU)."""

    def __init__(self, device, slot_bytes=64 << 20, slots=3):
        import torch
        self.torch, self.device = torch, torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.slot_bytes, self.h2d_bytes = slot_bytes, 0
        if self.cuda:
            self.stream = torch.cuda.Stream(self.device)
            self.ring = [torch.empty(slot_bytes, dtype=torch.uint8).pin_memory() for _ in range(slots)]
            self.free_at = [None] * slots
            self.next = 0

    def copy(self, dst, src_bytes):
        torch = self.torch
        flat = dst.view(-1).view(torch.uint8)
        if len(src_bytes) != flat.numel():
            raise IngestError("TensorsDict", f"{len(src_bytes)} bytes for a tensor of {flat.numel()}")
        if not self.cuda:
            flat.copy_(_as_u8(torch, src_bytes))
            return
        for o in range(0, len(src_bytes), self.slot_bytes):
            n = min(self.slot_bytes, len(src_bytes) - o)
            i = self.next
            self.next = (i + 1) % len(self.ring)
            if self.free_at[i] is not None:
                self.free_at[i].synchronize()                  # the slot's previous transfer has left it
            self.ring[i][:n].copy_(_as_u8(torch, src_bytes[o:o + n]))   # page cache -> pinned
            with torch.cuda.stream(self.stream):
                flat[o:o + n].copy_(self.ring[i][:n], non_blocking=True)
                self.free_at[i] = torch.cuda.Event()
                self.free_at[i].record(self.stream)
            self.h2d_bytes += n

    def flush(self):
        if self.cuda:
            self.stream.synchronize()


def load_llama(reader, params, copier=None):
    """Fill `params` (the structure of llama_step.init_weights) from a TensorsDir / PickleDir.  Shapes and dtypes must
    agree exactly (the reference asserts the same through its cell types).  Returns {parameter path: key}."""
    n_layers = len(params["layers"])
    matches = match_llama(n_layers, reader.clone_keys())
    flat = {"embed": params["embed"], "lm_head": params["lm_head"], "head_norm": params["head_norm"]}
    for i, L in enumerate(params["layers"]):
        for k, v in L.items():
            flat[f"layers.{i}.{k}"] = v
    missing = sorted(set(flat) - set(matches))
    if missing:
        raise IngestError("Path", f"no checkpoint tensor for {missing[:4]}{'...' if len(missing) > 4 else ''}")
    copier = copier or StagedCopier(params["embed"].device)
    for path, dst in flat.items():
        tag, shape, view = reader.get(matches[path])
        if tuple(shape) != tuple(dst.shape) or _torch_dtype(tag) != dst.dtype:
            raise IngestError("TensorsDict", f"{matches[path]}: {tag}{list(shape)} in file, "
                                             f"{dst.dtype}{list(dst.shape)} in the model")
        copier.copy(dst, view)
    copier.flush()
    return matches
