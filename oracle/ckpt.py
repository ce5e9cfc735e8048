"""Reader/writer for GradCraft's tensor checkpoint files (test infrastructure).

Layout, little endian, as written by save_tensor_checkpoint (gradc/nn/utils/checkpoint.hpp:12-36):
u32 sizeof(T); i64 tensor count; then per tensor: i64 name length, name bytes, i64 rank,
i64 dims[rank], i64 payload bytes, raw payload.
"""
import struct

import numpy as np


def save(path, tensors, dtype=np.float32):
    dtype = np.dtype(dtype)
    with open(path, "wb") as f:
        f.write(struct.pack("<I", dtype.itemsize))
        f.write(struct.pack("<q", len(tensors)))
        for name, arr in tensors.items():
            a = np.ascontiguousarray(np.asarray(arr, dtype=dtype))
            nb = name.encode()
            f.write(struct.pack("<q", len(nb)))
            f.write(nb)
            f.write(struct.pack("<q", a.ndim))
            f.write(struct.pack("<%dq" % a.ndim, *a.shape))
            f.write(struct.pack("<q", a.nbytes))
            f.write(a.tobytes())


def load(path, dtype=np.float32):
    dtype = np.dtype(dtype)
    out = {}
    with open(path, "rb") as f:
        (tag,) = struct.unpack("<I", f.read(4))
        if tag != dtype.itemsize:
            raise ValueError("checkpoint element size %d does not match dtype %s" % (tag, dtype))
        (n,) = struct.unpack("<q", f.read(8))
        for _ in range(n):
            (ln,) = struct.unpack("<q", f.read(8))
            name = f.read(ln).decode()
            (rank,) = struct.unpack("<q", f.read(8))
            shape = struct.unpack("<%dq" % rank, f.read(8 * rank)) if rank else ()
            (nbytes,) = struct.unpack("<q", f.read(8))
            out[name] = np.frombuffer(f.read(nbytes), dtype=dtype).reshape(shape).copy()
    return out
