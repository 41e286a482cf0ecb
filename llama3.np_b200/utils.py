"""Weight IO - the reference's `utils.py:4-5` surface (`load_parameters = np.load`)."""
import numpy as np


def load_parameters(model_path):
    """Return a mapping key -> ndarray.  Accepts a path to an `.npz` (as the reference
    does) or an already-loaded mapping (extension: 8B-shaped synthetic weights are
    impractical as a file)."""
    if isinstance(model_path, (str, bytes)) or hasattr(model_path, "__fspath__"):
        return np.load(model_path)
    return model_path


def checkpoint_digest(model_path, chunk: int = 1 << 24) -> str:
    """sha256 (hex) of the checkpoint FILE's bytes: the key of the packed device-layout cache
    (`Llama(..., cache_dir=...)`), so an edited or replaced `.npz` can never be served from a stale pack."""
    import hashlib
    h = hashlib.sha256()
    with open(model_path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def packed_cache_path(cache_dir, digest: str, dtype: str, tp_rank: int = 0, tp_world: int = 1) -> str:
    """Where the pack of one (checkpoint, dtype, tensor-parallel placement) lives inside `cache_dir`."""
    import os
    kind = "bf16" if dtype in ("bfloat16", "bf16") else "f32"
    return os.path.join(os.fspath(cache_dir), f"{digest[:40]}.{kind}.tp{tp_rank}of{tp_world}.l3pack")


def read_safetensors(path) -> dict:
    """Tensors of a `.safetensors` file as NumPy arrays, without any library: the file is an 8-byte
    little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets) and the data.
    bfloat16 comes back as float32 (exact: bf16 is the top half of an fp32), integer tables keep their type."""
    import json
    import struct
    kinds = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64,
             "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            half = np.frombuffer(blob, dtype="<u2", count=(hi - lo) // 2, offset=lo)
            arr = (half.astype(np.uint32) << 16).view(np.float32)
        elif meta["dtype"] in kinds:
            dt = np.dtype(kinds[meta["dtype"]]).newbyteorder("<")
            arr = np.frombuffer(blob, dtype=dt, count=(hi - lo) // dt.itemsize, offset=lo)
        else:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        out[name] = arr.reshape(shape)
    return out
