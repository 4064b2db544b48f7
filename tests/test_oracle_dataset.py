"""The input-pipeline oracle (oracle/dataset.py) against the reference's own loader test and the published
known answers of its generator.  Runs without a GPU."""
import struct

import numpy as np
import pytest

from oracle import dataset as od


def mock():
    """The mock dataset of the reference's test (src/dataset.zig:228-253): 12 samples of 2 values, value = index."""
    return np.arange(24, dtype=np.float32).reshape(12, 2), np.arange(12, dtype=np.uint8)


def replay_reference_loader_test(make_loader, buffers, read):
    """src/dataset.zig:255-300, statement by statement, for any loader with the mirrored interface."""
    loader = make_loader(batch_size=5, shuffle=False, drop_last=False)
    x_buf, y_buf = buffers(5, 2)
    assert loader.next_into(x_buf, y_buf) == 5
    x, y = read(x_buf, y_buf)
    assert x.flat[0] == 0.0 and x.flat[1] == 1.0 and y[0] == 0 and y[4] == 4
    assert loader.next_into(x_buf, y_buf) == 5
    x, y = read(x_buf, y_buf)
    assert x.flat[0] == 10.0 and y[0] == 5
    assert loader.next_into(x_buf, y_buf) == 2
    x, y = read(x_buf, y_buf)
    assert x.flat[0] == 20.0 and y[0] == 10
    assert loader.next_into(x_buf, y_buf) is None
    loader.drop_last = True
    loader.reset()
    assert loader.next_into(x_buf, y_buf) == 5
    assert loader.next_into(x_buf, y_buf) == 5
    assert loader.next_into(x_buf, y_buf) is None


def test_reference_loader_test_on_the_oracle():
    images, labels = mock()
    replay_reference_loader_test(
        lambda **kw: od.DataLoader(images, labels, **kw),
        lambda b, d: (np.zeros((b, d), np.float32), np.zeros(b, np.uint8)),
        lambda x, y: (x, y))


def test_peek_next_batch_size():
    images, labels = mock()
    ld = od.DataLoader(images, labels, 5)
    x, y = np.zeros((5, 2), np.float32), np.zeros(5, np.uint8)
    sizes = []
    while True:
        sizes.append(ld.peek_next_batch_size())
        if ld.next_into(x, y) is None:
            break
    assert sizes == [5, 5, 2, 0]


def test_generator_known_answers():
    g = od.Xoshiro256(0)
    g.s = [1, 2, 3, 4]
    assert [g.next() for _ in range(6)] == [41943041, 58720359, 3588806011781223, 3591011842654386,
                                             9228616714210784205, 9973669472204895162]
    assert od.Xoshiro256(1234567).s == [6457827717110365317, 3203168211198807973, 9817491932198370423,
                                         4593380528125082431]


def test_bounded_draw_properties():
    g = od.Xoshiro256(7)
    for bound in (1, 2, 3, 10, 60000, (1 << 63) + 5):
        draws = [g.uint_less_than(bound) for _ in range(200)]
        assert all(0 <= d < bound for d in draws)
    counts = np.bincount([g.uint_less_than(6) for _ in range(60000)], minlength=6)
    assert counts.min() > 9500 and counts.max() < 10500


def test_shuffle_is_a_seeded_permutation():
    images, labels = np.zeros((1000, 1), np.float32), np.zeros(1000, np.uint8)
    a = od.DataLoader(images, labels, 10, shuffle=True)
    b = od.DataLoader(images, labels, 10, shuffle=True, seed=1337)
    c = od.DataLoader(images, labels, 10, shuffle=True, seed=1)
    assert a.indices == b.indices != c.indices
    assert sorted(a.indices) == list(range(1000)) and a.indices != list(range(1000))
    first = list(a.indices)
    a.reset()
    assert sorted(a.indices) == list(range(1000)) and a.indices != first


def test_idx_parsing():
    px = np.arange(2 * 3 * 4, dtype=np.uint8) * 10
    blob = struct.pack(">IIII", 0x803, 2, 3, 4) + px.tobytes()
    images, rows, cols = od.load_images(blob)
    assert (rows, cols) == (3, 4) and images.shape == (2, 12) and images.dtype == np.float32
    assert images[0, 0] == 0.0 and images[1, 11] == np.float32(230) / np.float32(255)
    assert od.load_images(struct.pack(">IIII", 0x803, 1, 1, 1) + b"\xff")[0][0, 0] == 1.0
    labels = od.load_labels(struct.pack(">II", 0x801, 3) + b"\x07\x00\x09")
    assert labels.tolist() == [7, 0, 9]
    with pytest.raises(ValueError, match="InvalidMagicNumber"):
        od.load_images(struct.pack(">IIII", 0x801, 1, 1, 1) + b"\x00")
    with pytest.raises(ValueError, match="InvalidMagicNumber"):
        od.load_labels(struct.pack(">II", 0x803, 1) + b"\x00")
    with pytest.raises(ValueError, match="EndOfStream"):
        od.load_images(struct.pack(">IIII", 0x803, 2, 2, 2) + b"\x00" * 7)
