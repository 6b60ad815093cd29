"""Model weights over safetensors files: key-addressed access to a checkpoint directory and the
load path onto the GPU (reference: src/ucode/ampstein/weights.uc, the `ws` object every model
builder takes; same method names and meaning).

Both on-disk layouts: <dir>/model.safetensors, or <dir>/model.safetensors.index.json whose
"weight_map" routes every key to a shard file. Files are memory-mapped; tensor() is a zero-copy
CPU view. gpu() uploads one tensor on first touch and caches it; upload() moves every tensor (or a
list of keys) in batches: the bytes of a batch are gathered into one of two pinned staging buffers
(this is where the file is actually read) and copied with ONE asynchronous transfer on a copy
stream into one device allocation, while the next batch is being gathered into the other buffer;
the tensors are views of those device allocations at 256-byte aligned offsets. For the EXL3
linears this is the whole load: trellis / suh / svh go to the device exactly as stored.

The format is the public safetensors layout: 8 bytes little-endian header length N, N bytes of JSON
{key: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the byte buffer."""
import builtins
import json
import mmap
import os
import struct

import numpy as np
import torch

INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"

_DTYPES = {
    "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "U16": (torch.int16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}


class _StFile:
    """One safetensors file: parsed header + a read-only memory map."""

    def __init__(self, path):
        self.path = path
        self._f = builtins.open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError("weights: %s is not a safetensors file" % path)
        (n,) = struct.unpack("<Q", head)
        size = os.fstat(self._f.fileno()).st_size
        if n < 2 or 8 + n > size:
            raise ValueError("weights: %s: bad header length" % path)
        meta = json.loads(self._f.read(n).decode("utf-8"))
        self.base = 8 + n
        self.entries = {}
        for key, e in meta.items():
            if key == "__metadata__":
                continue
            if e["dtype"] not in _DTYPES:
                raise ValueError("weights: %s: %s has unsupported dtype %s" % (path, key, e["dtype"]))
            b, end = e["data_offsets"]
            count = 1
            for d in e["shape"]:
                count *= int(d)
            if end - b != count * _DTYPES[e["dtype"]][1] or self.base + end > size or b < 0:
                raise ValueError("weights: %s: %s has inconsistent offsets" % (path, key))
            self.entries[key] = (e["dtype"], tuple(int(d) for d in e["shape"]), int(b), int(end))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def raw(self, key):
        """uint8 numpy view of the tensor's bytes inside the map (zero-copy)."""
        _, _, b, e = self.entries[key]
        return np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self.base + b)


class WeightSet:
    def __init__(self, model_dir, only_file=None):
        self.dir = model_dir
        self._files = {}                  # file name -> _StFile (opened lazily)
        self._map = None                  # sharded: key -> file name
        self._single = None
        self._gpu = {}                    # (key, device index) -> CUDA tensor
        if only_file:
            self._single = only_file
        elif os.path.exists(os.path.join(model_dir, INDEX_NAME)):
            with builtins.open(os.path.join(model_dir, INDEX_NAME)) as f:
                idx = json.load(f)
            self._map = idx.get("weight_map")
            if not self._map:
                raise ValueError("weights: %s has no weight_map" % INDEX_NAME)
        else:
            self._single = SINGLE_NAME
            if not os.path.exists(os.path.join(model_dir, SINGLE_NAME)):
                raise FileNotFoundError("weights: neither %s nor %s in %s" % (INDEX_NAME, SINGLE_NAME, model_dir))

    # ---- lookup ----
    def _file(self, name):
        f = self._files.get(name)
        if f is None:
            f = self._files[name] = _StFile(os.path.join(self.dir, name))
        return f

    def _where(self, key):
        if self._map is not None:
            name = self._map.get(key)
            if name is None:
                raise KeyError("weights: no tensor %s" % key)
            f = self._file(name)
        else:
            f = self._file(self._single)
        if key not in f.entries:
            raise KeyError("weights: no tensor %s" % key)
        return f

    def has(self, key):
        if self._map is not None:
            return key in self._map
        return key in self._file(self._single).entries

    def keys(self):
        return sorted(self._map) if self._map is not None else sorted(self._file(self._single).entries)

    def info(self, key):
        dt, shape, _, _ = self._where(key).entries[key]
        return {"shape": list(shape), "dtype": dt}

    # ---- host views ----
    def tensor(self, key):
        """CPU tensor over the memory map (zero-copy, read-only data: clone before writing)."""
        f = self._where(key)
        dt, shape, _, _ = f.entries[key]
        raw = f.raw(key)
        if raw.size == 0:
            return torch.empty(shape, dtype=_DTYPES[dt][0])
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")               # (torch warns about non-writable numpy memory)
            t = torch.from_numpy(raw)
        return t.view(_DTYPES[dt][0]).view(shape)

    def fp16(self, key):
        return self.tensor(key).to(torch.float16)

    # ---- device ----
    def gpu(self, key, dev=0):
        """CUDA tensor of `key` on device `dev` (cached; uploaded on first touch)."""
        dev = 0 if dev is None else int(dev)
        t = self._gpu.get((key, dev))
        if t is None:
            self.upload(dev, [key])
            t = self._gpu[(key, dev)]
        return t

    def gpu16(self, key, dev=0):
        t = self.gpu(key, dev)
        return t if t.dtype == torch.float16 else t.to(torch.float16)

    def upload(self, dev=0, keys=None, batch_bytes=256 << 20):
        """Moves `keys` (default: every tensor not yet on device `dev`) to the GPU in batches of up to
        batch_bytes: gather into pinned memory, one asynchronous copy per batch on a copy stream,
        double-buffered. Returns the number of bytes moved."""
        if not torch.cuda.is_available():
            raise RuntimeError("weights.upload: no CUDA device (host tensors come from tensor())")
        dev = 0 if dev is None else int(dev)
        todo = [k for k in (self.keys() if keys is None else keys) if (k, dev) not in self._gpu]
        if not todo:
            return 0
        batches, cur, cur_bytes = [], [], 0
        for k in todo:
            f = self._where(k)
            _, _, b, e = f.entries[k]
            n = (e - b + 255) & ~255
            if cur and cur_bytes + n > batch_bytes:
                batches.append((cur, cur_bytes))
                cur, cur_bytes = [], 0
            cur.append((k, f, cur_bytes, e - b))
            cur_bytes += n
        if cur:
            batches.append((cur, cur_bytes))
        device = torch.device("cuda", dev)
        stage_bytes = max(nb for _, nb in batches)
        moved = 0
        with torch.cuda.device(device):
            stage = [torch.empty(stage_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(min(2, len(batches)))]
            done = [None] * len(stage)
            copy_stream = torch.cuda.Stream()
            for i, (items, nbytes) in enumerate(batches):
                s = i % len(stage)
                if done[s] is not None:
                    done[s].synchronize()                 # the copy that last used this staging buffer has finished
                host = stage[s].numpy()
                for k, f, off, n in items:
                    if n:
                        host[off:off + n] = f.raw(k)      # the file read happens here
                dbuf = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
                with torch.cuda.stream(copy_stream):
                    dbuf[:nbytes].copy_(stage[s][:nbytes], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                done[s] = ev
                for k, f, off, n in items:
                    dt, shape, _, _ = f.entries[k]
                    self._gpu[(k, dev)] = dbuf[off:off + n].view(_DTYPES[dt][0]).view(shape) if n else \
                        torch.empty(shape, dtype=_DTYPES[dt][0], device=device)
                moved += nbytes
            # the tensors are used on other streams: make the current stream wait for the copies
            torch.cuda.current_stream().wait_stream(copy_stream)
        return moved


def open(model_dir, only_file=None):      # noqa: A001  (the reference's name: weights.open)
    return WeightSet(model_dir, only_file)


def save_file(tensors, path, metadata=None):
    """Writes a safetensors file from {key: CPU tensor} (used by the tests and by tools that build
    synthetic checkpoints; not part of the reference's runtime)."""
    names = {v[0]: k for k, v in _DTYPES.items() if k != "U16"}
    header, blobs, off = {}, [], 0
    for key in sorted(tensors):
        t = tensors[key].detach().contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[key] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * ((8 - len(h) % 8) % 8)
    with builtins.open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
