"""Python view of the host mirror's models (include/znn_host.h, znn_model_*): the
reference's example programs (MLP, CNN, transformer block, GPT) with their
training step, run entirely by the C++ host mirror over the CUDA kernels."""
import ctypes as C

import numpy as np

from ._lib import lib

KINDS = {"mlp": 1, "cnn_ref": 2, "cnn_padded": 3, "block": 4, "gpt": 5}


class Model:
    def __init__(self, kind, dims=(), arena_bytes=1 << 30):
        self.kind = kind
        d = (C.c_longlong * max(1, len(dims)))(*dims)
        h = C.c_void_p()
        lib().call("znn_model_create", KINDS[kind], d, len(dims), arena_bytes, C.byref(h))
        self.h = h
        n = C.c_int()
        lib().call("znn_model_param_count", self.h, C.byref(n))
        self.params = []   # (name, shape, offset, fan_in)
        for i in range(n.value):
            name = C.create_string_buffer(128)
            dims8 = (C.c_longlong * 8)()
            rank, off, fan = C.c_int(), C.c_longlong(), C.c_longlong()
            lib().call("znn_model_param_info", self.h, i, name, 128, dims8, C.byref(rank), C.byref(off), C.byref(fan))
            self.params.append((name.value.decode(), tuple(int(dims8[k]) for k in range(rank.value)), off.value, fan.value))
        t = C.c_longlong()
        lib().call("znn_model_total_floats", self.h, C.byref(t))
        self.total = t.value

    def close(self):
        if self.h:
            lib().call("znn_model_destroy", self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters as dicts name -> array
    def _pack(self, P):
        slab = np.zeros(self.total, np.float32)
        for name, shape, off, _ in self.params:
            a = np.asarray(P[name], np.float32)
            assert a.size == int(np.prod(shape)), (name, a.shape, shape)
            slab[off:off + a.size] = a.reshape(-1)
        return slab

    def _unpack(self, slab):
        return {name: slab[off:off + int(np.prod(shape))].reshape(shape).copy() for name, shape, off, _ in self.params}

    def set_params(self, P):
        slab = self._pack(P)
        lib().call("znn_model_set_params", self.h, slab.ctypes.data)

    def _get(self, fn):
        slab = np.empty(self.total, np.float32)
        lib().call(fn, self.h, slab.ctypes.data)
        return self._unpack(slab)

    def save(self, path):
        """Checkpoint in the reference's safetensors-style layout (src/nn.zig:268-303)."""
        lib().call("znn_model_save", self.h, str(path).encode())

    def load(self, path):
        lib().call("znn_model_load", self.h, str(path).encode())

    def save_optimizer(self, path):
        """The SGD velocities in a second file of the same layout (resume = load + load_optimizer)."""
        lib().call("znn_model_save_optimizer", self.h, str(path).encode())

    def load_optimizer(self, path):
        lib().call("znn_model_load_optimizer", self.h, str(path).encode())

    def get_params(self): return self._get("znn_model_get_params")
    def get_grads(self): return self._get("znn_model_get_grads")
    def get_velocities(self): return self._get("znn_model_get_velocities")

    def set_option(self, key, value):
        lib().call("znn_model_set_option", self.h, key.encode(), float(value))
        if key == "targets_u8":
            self._targets_u8 = bool(value)

    def train_step(self, x, targets, seq=0, read_loss=True):
        x = np.ascontiguousarray(x, np.float32)
        t = np.ascontiguousarray(targets, np.uint8 if getattr(self, "_targets_u8", False) else np.int32)
        batch = x.shape[0]
        loss = C.c_float()
        lib().call("znn_model_train_step", self.h, x.ctypes.data, t.ctypes.data, batch, seq, 0,
                   C.byref(loss) if read_loss else None)
        return loss.value if read_loss else None

    def train_step_device(self, x_ptr, t_ptr, batch, seq=0, loss_ptr=None):
        lib().call("znn_model_train_step", self.h, x_ptr, t_ptr, batch, seq, 1, loss_ptr)

    def evaluate(self, x, labels):
        """(loss, accuracy) of one batch: host arrays, labels as bytes."""
        x = np.ascontiguousarray(x, np.float32)
        y = np.ascontiguousarray(labels, np.uint8)
        loss, acc = C.c_float(), C.c_float()
        lib().call("znn_model_evaluate", self.h, x.ctypes.data, y.ctypes.data, x.shape[0], 0, C.byref(loss), C.byref(acc))
        return loss.value, acc.value

    def evaluate_device(self, x_ptr, y_ptr, batch):
        loss, acc = C.c_float(), C.c_float()
        lib().call("znn_model_evaluate", self.h, x_ptr, y_ptr, batch, 1, C.byref(loss), C.byref(acc))
        return loss.value, acc.value

    def forward(self, x, seq=0, classes=None):
        x = np.ascontiguousarray(x, np.float32)
        batch = x.shape[0]
        rows = batch * (seq if seq else 1)
        out = np.empty((rows, classes), np.float32)
        lib().call("znn_model_forward", self.h, x.ctypes.data, batch, seq, 0, out.ctypes.data)
        return out

    def block_fwd_bwd(self, x, dy):
        x = np.ascontiguousarray(x, np.float32)
        dy = np.ascontiguousarray(dy, np.float32)
        B, T, _ = x.shape
        y, dx = np.empty_like(x), np.empty_like(x)
        lib().call("znn_model_block_fwd_bwd", self.h, x.ctypes.data, dy.ctypes.data, B, T, y.ctypes.data, dx.ctypes.data)
        return y, dx

    def block_fwd_bwd_device(self, x_ptr, dy_ptr, B, T, y_ptr, dx_ptr):
        """Device pointers in and out; returns at once (work is queued on the thread's stream)."""
        lib().call("znn_model_block_fwd_bwd_device", self.h, x_ptr, dy_ptr, B, T, y_ptr, dx_ptr)

    def greedy_decode(self, prompts, n_new):
        p = np.ascontiguousarray(prompts, np.float32)
        out = np.empty((p.shape[0], n_new), np.float32)
        lib().call("znn_model_greedy_decode", self.h, p.ctypes.data, p.shape[0], p.shape[1], n_new, out.ctypes.data)
        return out

    def greedy_decode_kv(self, prompts, n_new):
        """Greedy decode with a key/value cache (same tokens as greedy_decode while the window does not slide)."""
        p = np.ascontiguousarray(prompts, np.float32)
        out = np.empty((p.shape[0], n_new), np.float32)
        lib().call("znn_model_greedy_decode_kv", self.h, p.ctypes.data, p.shape[0], p.shape[1], n_new, out.ctypes.data)
        return out

    def graph_replays(self):
        n = C.c_longlong()
        lib().call("znn_model_graph_replays", self.h, C.byref(n))
        return n.value

    def last_step_ops(self):
        n = C.c_int()
        lib().call("znn_model_last_step_ops", self.h, C.byref(n))
        return n.value

    def arena_high_water(self):
        b = C.c_longlong()
        lib().call("znn_model_arena_high_water", self.h, C.byref(b))
        return b.value
