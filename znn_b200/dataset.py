"""Input pipeline with the dataset resident in device memory: mirror of the reference's src/dataset.zig.

`load_dataset` = loadDataset (src/dataset.zig:108-124), `DataLoader` = DataLoader (src/dataset.zig:132-223) with the
same names and meaning: `peek_next_batch_size`, `next_into` (returns the batch size, or None where the reference
returns null), `reset`, the `drop_last` attribute.  All work is done by the C ABI (znn_dataset_load_idx,
znn_loader_*); a batch is one gather launch on the device.
"""
import ctypes as C

import numpy as np

from ._lib import lib
from . import ops


class _Borrowed:
    """Device memory handed out by the library; freed with znn_free."""

    def __init__(self, ptr):
        self.ptr = ptr

    def free(self):
        if self.ptr:
            lib().call("znn_free", self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Dataset:
    """images: fp32 [num_images, rows*cols] in [0, 1]; labels: u8 [num_items]; both on the device."""

    def __init__(self, images, labels, num_images, rows, cols, num_items):
        self.images, self.labels = images, labels
        self.num_images, self.rows, self.cols, self.num_items = num_images, rows, cols, num_items

    @classmethod
    def from_arrays(cls, images, labels, rows=None, cols=1):
        """Already-converted fp32 samples (as the reference's own test builds them) and u8 labels."""
        ops._ensure()
        images = np.ascontiguousarray(images, np.float32)
        labels = np.ascontiguousarray(labels, np.uint8)
        n = images.shape[0]
        dim = int(images.size // max(n, 1))
        rows = dim // cols if rows is None else rows
        return cls(ops.DevBuf.from_host(images), ops.DevBuf.from_host(labels), n, rows, cols, labels.size)

    def images_to_host(self):
        out = np.empty((self.num_images, self.rows * self.cols), np.float32)
        if out.nbytes:
            lib().call("znn_memcpy_d2h", out.ctypes.data, self.images.ptr, out.nbytes)
        return out


def load_dataset(images_path, labels_path):
    ops._ensure()
    img, lab = C.c_void_p(), C.c_void_p()
    n, r, c, items = C.c_uint(), C.c_uint(), C.c_uint(), C.c_uint()
    lib().call("znn_dataset_load_idx", str(images_path).encode(), str(labels_path).encode(), C.byref(img), C.byref(lab),
               C.byref(n), C.byref(r), C.byref(c), C.byref(items))
    return Dataset(_Borrowed(img.value), _Borrowed(lab.value), n.value, r.value, c.value, items.value)


class DataLoader:
    def __init__(self, dataset, batch_size, shuffle=False, seed=None, drop_last=False):
        self.dataset, self.batch_size = dataset, int(batch_size)
        self.input_dim = dataset.rows * dataset.cols
        h = C.c_void_p()
        lib().call("znn_loader_create", dataset.images.ptr, dataset.labels.ptr, dataset.num_images, self.input_dim,
                   self.batch_size, int(shuffle), int(drop_last), -1 if seed is None else int(seed), C.byref(h))
        self._h = h.value
        self._drop_last = bool(drop_last)

    @property
    def drop_last(self):
        return self._drop_last

    @drop_last.setter
    def drop_last(self, v):
        lib().call("znn_loader_set_drop_last", self._h, int(bool(v)))
        self._drop_last = bool(v)

    def reset(self):
        lib().call("znn_loader_reset", self._h)

    def peek_next_batch_size(self):
        n = C.c_size_t()
        lib().call("znn_loader_peek_next_batch_size", self._h, C.byref(n))
        return n.value

    def next_into(self, x_dest, y_dest):
        """x_dest, y_dest: device buffers (DevBuf) of batch_size*input_dim floats and batch_size bytes."""
        n = C.c_size_t()
        lib().call("znn_loader_next_into", self._h, x_dest.ptr, y_dest.ptr, C.byref(n))
        return n.value or None

    def indices(self):
        out = np.empty(self.dataset.num_images, np.int32)
        lib().call("znn_loader_indices", self._h, out.ctypes.data, out.size)
        return out

    def close(self):
        if self._h:
            lib().call("znn_loader_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
