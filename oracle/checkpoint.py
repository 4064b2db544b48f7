"""Test infrastructure: the reference's checkpoint layout restated in Python (src/nn.zig:173-303 saveModel,
:354-455 loadModel).  Only tests may import this.

File = 8-byte little-endian u64 header length | JSON header | fp32 data.  The header is
{"name":{"dtype":"F32","shape":[d0,d1],"data_offsets":[start,end]},...} with no spaces, entries in the order of the
model's struct fields (src/nn.zig:193-236), padded with spaces to a multiple of 8 (:283-288); the data follow back to
back in the same order (:238-264).
"""
import json
import struct

import numpy as np


def header_bytes(named_shapes):
    """named_shapes: [(name, shape)] in parameter order."""
    parts, off = [], 0
    for name, shape in named_shapes:
        n = int(np.prod(shape)) * 4
        dims = ",".join(str(int(d)) for d in shape)
        parts.append('"%s":{"dtype":"F32","shape":[%s],"data_offsets":[%d,%d]}' % (name, dims, off, off + n))
        off += n
    h = "{" + ",".join(parts) + "}"
    h += " " * ((8 - len(h) % 8) % 8)
    return h.encode()


def save(path, named_arrays):
    """named_arrays: [(name, float32 array)] in parameter order."""
    h = header_bytes([(n, a.shape) for n, a in named_arrays])
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for _, a in named_arrays:
            f.write(np.ascontiguousarray(a, np.float32).tobytes())


def load(path, named_shapes):
    """Returns {name: array}; checks what loadTensorData checks (:384-455)."""
    with open(path, "rb") as f:
        (hl,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(hl).decode())
        data = f.read()
    out, current = {}, 0
    for name, shape in named_shapes:
        m = meta[name]
        assert m["dtype"] == "F32", name
        assert tuple(m["shape"]) == tuple(shape), (name, m["shape"], shape)
        s, e = m["data_offsets"]
        assert e - s == int(np.prod(shape)) * 4 and s >= current, name
        out[name] = np.frombuffer(data[s:e], np.float32).reshape(shape).copy()
        current = e
    return out
