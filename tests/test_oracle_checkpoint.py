"""The checkpoint layout restated from src/nn.zig:173-455 (oracle/checkpoint.py): header text, padding, offsets."""
import struct

import numpy as np

from oracle import checkpoint


def test_header_layout_and_round_trip(tmp_path):
    shapes = [("fc1.weight", (3, 2)), ("fc1.bias", (1, 2)), ("h.0.ln.weight", (5,))]
    h = checkpoint.header_bytes(shapes)
    assert len(h) % 8 == 0 and h.rstrip(b" ").endswith(b"}")
    assert h.startswith(b'{"fc1.weight":{"dtype":"F32","shape":[3,2],"data_offsets":[0,24]},"fc1.bias":{"dtype":"F32",'
                        b'"shape":[1,2],"data_offsets":[24,32]},"h.0.ln.weight":{"dtype":"F32","shape":[5],"data_offsets":[32,52]}}')
    r = np.random.default_rng(0)
    arrays = [(n, r.standard_normal(s).astype(np.float32)) for n, s in shapes]
    path = tmp_path / "m.safetensors"
    checkpoint.save(path, arrays)
    raw = path.read_bytes()
    (hl,) = struct.unpack("<Q", raw[:8])
    assert hl == len(h) and raw[8:8 + hl] == h and len(raw) == 8 + hl + 52
    back = checkpoint.load(path, shapes)
    for n, a in arrays:
        np.testing.assert_array_equal(back[n], a)
