"""CPU restatement of the reference's input pipeline (src/dataset.zig).  TEST INFRASTRUCTURE ONLY: the checker
of the device loader, never the thing shipped or measured.

Pinned: batch sizes, sample order without shuffling, drop_last and reset follow the reference's own test
"DataLoader basic functionality" (src/dataset.zig:225-300), which tests/test_oracle_dataset.py replays.
The generator is pinned on the published known-answer sequences of its two algorithms (xoshiro256++ from state
1,2,3,4; SplitMix64 from seed 1234567), also replayed there.
Parity unpinned: the ORDER a shuffle produces, as far as it depends on the bounded draw.  The reference's toolchain
draws with std.Random.DefaultPrng (xoshiro256++ seeded through SplitMix64) and intRangeLessThan (Lemire's
multiply-and-reject), restated here from the published algorithm; the reference holds no golden vector for a shuffled
order and no Zig toolchain is available to produce one.
"""
import struct

import numpy as np

M64 = (1 << 64) - 1


def load_images(blob):
    """loadImages (src/dataset.zig:23-71): big-endian header, magic 0x803, pixel / 255.0 in fp32."""
    if len(blob) < 16:
        raise ValueError("EndOfStream")
    magic, n, rows, cols = struct.unpack(">IIII", blob[:16])
    if magic != 0x803:
        raise ValueError("InvalidMagicNumber")
    count = n * rows * cols
    if len(blob) - 16 < count:
        raise ValueError("EndOfStream")
    px = np.frombuffer(blob, np.uint8, count, 16)
    return (px.astype(np.float32) / np.float32(255.0)).reshape(n, rows * cols), rows, cols


def load_labels(blob):
    """loadLabels (src/dataset.zig:73-106)."""
    if len(blob) < 8:
        raise ValueError("EndOfStream")
    magic, n = struct.unpack(">II", blob[:8])
    if magic != 0x801:
        raise ValueError("InvalidMagicNumber")
    if len(blob) - 8 < n:
        raise ValueError("EndOfStream")
    return np.frombuffer(blob, np.uint8, n, 8).copy()


class Xoshiro256:
    def __init__(self, seed):
        x, self.s = seed & M64, []
        for _ in range(4):
            x = (x + 0x9E3779B97F4A7C15) & M64
            z = x
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(v, k):
        return ((v << k) | (v >> (64 - k))) & M64

    def next(self):
        s = self.s
        r = (self._rotl((s[0] + s[3]) & M64, 23) + s[0]) & M64
        t = (s[1] << 17) & M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return r

    def uint_less_than(self, less_than):
        m = self.next() * less_than
        low = m & M64
        if low < less_than:
            t = (-less_than) & M64
            if t >= less_than:
                t -= less_than
                if t >= less_than:
                    t %= less_than
            while low < t:
                m = self.next() * less_than
                low = m & M64
        return m >> 64


class DataLoader:
    """DataLoader (src/dataset.zig:132-223) over numpy arrays."""

    def __init__(self, images, labels, batch_size, shuffle=False, seed=None, drop_last=False):
        self.images, self.labels = images, labels
        self.batch_size, self.shuffle, self.drop_last = batch_size, shuffle, drop_last
        self.indices = list(range(images.shape[0]))
        self.current_index = 0
        self.prng = Xoshiro256(1337 if seed is None else seed)
        if shuffle:
            self.shuffle_indices()

    def shuffle_indices(self):
        i = len(self.indices) - 1
        while i > 0:
            j = self.prng.uint_less_than(i + 1)
            self.indices[i], self.indices[j] = self.indices[j], self.indices[i]
            i -= 1

    def reset(self):
        self.current_index = 0
        if self.shuffle:
            self.shuffle_indices()

    def peek_next_batch_size(self):
        n = len(self.indices)
        if self.current_index >= n:
            return 0
        remaining = n - self.current_index
        if self.drop_last and remaining < self.batch_size:
            return 0
        return min(self.batch_size, remaining)

    def next_into(self, x_dest, y_dest):
        take = self.peek_next_batch_size()
        if take == 0:
            return None
        for j in range(take):
            idx = self.indices[self.current_index + j]
            x_dest[j, :] = self.images[idx, :]
            y_dest[j] = self.labels[idx]
        self.current_index += take
        return take
