"""The device-resident input pipeline (znn_dataset_load_idx, znn_loader_*, znn_batch_gather, znn_pixels_to_unit)
against the CPU oracle of src/dataset.zig.  Bit-exact: the work is byte copies and one IEEE division per pixel."""
import struct

import numpy as np
import pytest

from oracle import dataset as od
from test_oracle_dataset import mock, replay_reference_loader_test

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ds():
    from znn_b200 import ops, dataset
    ops.init(0)
    return dataset


def dev_buffers(b, d):
    from znn_b200 import ops
    return ops.DevBuf(b * d * 4), ops.DevBuf(b)


def dev_read(shape_b, shape_d):
    return lambda x, y: (x.to_host((shape_b, shape_d)), y.to_host((shape_b,), np.uint8))


def test_reference_loader_test_on_the_device(ds):
    images, labels = mock()
    data = ds.Dataset.from_arrays(images, labels)
    replay_reference_loader_test(lambda **kw: ds.DataLoader(data, **kw), dev_buffers, dev_read(5, 2))


def test_pixels_to_unit_every_byte_value(ds):
    from znn_b200 import ops
    from znn_b200._lib import lib
    for n, shift in ((256, 0), (1021, 0), (4096 + 3, 1)):            # shift = 1: source not 4-byte aligned
        px = (np.arange(n + shift, dtype=np.uint32) * 37 % 256).astype(np.uint8)
        d_px, d_out = ops.DevBuf.from_host(px), ops.DevBuf(n * 4)
        lib().call("znn_pixels_to_unit", d_px.ptr + shift, d_out.ptr, n)
        want = px[shift:].astype(np.float32) / np.float32(255.0)
        np.testing.assert_array_equal(d_out.to_host((n,)), want)


@pytest.mark.parametrize("input_dim", [1, 3, 784, 1030])
@pytest.mark.parametrize("shuffle,seed", [(False, None), (True, None), (True, 99)])
def test_epochs_match_oracle(ds, input_dim, shuffle, seed):
    r = np.random.default_rng(input_dim)
    n, bs = 1003, 64
    images = r.standard_normal((n, input_dim), np.float32)
    labels = r.integers(0, 256, n).astype(np.uint8)
    data = ds.Dataset.from_arrays(images, labels)
    dev = ds.DataLoader(data, bs, shuffle=shuffle, seed=seed)
    ref = od.DataLoader(images, labels, bs, shuffle=shuffle, seed=seed)
    x_dev, y_dev = dev_buffers(bs, input_dim)
    for epoch in range(3):
        np.testing.assert_array_equal(dev.indices(), np.asarray(ref.indices, np.int32))
        while True:
            x_ref, y_ref = np.zeros((bs, input_dim), np.float32), np.zeros(bs, np.uint8)
            assert dev.peek_next_batch_size() == ref.peek_next_batch_size()
            got, want = dev.next_into(x_dev, y_dev), ref.next_into(x_ref, y_ref)
            assert got == want
            if got is None:
                break
            np.testing.assert_array_equal(x_dev.to_host((bs, input_dim))[:got], x_ref[:got])
            np.testing.assert_array_equal(y_dev.to_host((bs,), np.uint8)[:got], y_ref[:got])
        if epoch == 1:
            dev.drop_last = ref.drop_last = True
        dev.reset()
        ref.reset()


def test_gather_without_labels_and_unaligned_destination(ds):
    from znn_b200 import ops
    from znn_b200._lib import lib
    r = np.random.default_rng(2)
    images = r.standard_normal((50, 8), np.float32)
    idx = r.integers(0, 50, 20).astype(np.int32)
    d_img, d_idx = ops.DevBuf.from_host(images), ops.DevBuf.from_host(idx)
    d_out = ops.DevBuf((20 * 8 + 1) * 4)
    lib().call("znn_batch_gather", d_img.ptr, None, d_idx.ptr, d_out.ptr + 4, None, 20, 8, 50)   # dst 4-byte aligned only
    np.testing.assert_array_equal(d_out.to_host((20 * 8 + 1,))[1:].reshape(20, 8), images[idx])
    with pytest.raises(RuntimeError):
        lib().call("znn_batch_gather", d_img.ptr, None, d_idx.ptr, d_out.ptr, d_idx.ptr, 20, 8, 50)


def test_load_idx_files(ds, tmp_path):
    r = np.random.default_rng(4)
    n, rows, cols = 37, 28, 28
    px = r.integers(0, 256, n * rows * cols).astype(np.uint8)
    lab = r.integers(0, 10, n).astype(np.uint8)
    img_blob = struct.pack(">IIII", 0x803, n, rows, cols) + px.tobytes()
    lab_blob = struct.pack(">II", 0x801, n) + lab.tobytes()
    (tmp_path / "img").write_bytes(img_blob)
    (tmp_path / "lab").write_bytes(lab_blob)
    data = ds.load_dataset(tmp_path / "img", tmp_path / "lab")
    assert (data.num_images, data.rows, data.cols, data.num_items) == (n, rows, cols, n)
    want, _, _ = od.load_images(img_blob)
    np.testing.assert_array_equal(data.images_to_host(), want)
    loader = ds.DataLoader(data, 16, shuffle=True, seed=5)
    ref = od.DataLoader(want, od.load_labels(lab_blob), 16, shuffle=True, seed=5)
    x_dev, y_dev = dev_buffers(16, rows * cols)
    x_ref, y_ref = np.zeros((16, rows * cols), np.float32), np.zeros(16, np.uint8)
    assert loader.next_into(x_dev, y_dev) == ref.next_into(x_ref, y_ref) == 16
    np.testing.assert_array_equal(x_dev.to_host((16, rows * cols)), x_ref)
    np.testing.assert_array_equal(y_dev.to_host((16,), np.uint8), y_ref)

    (tmp_path / "bad").write_bytes(struct.pack(">IIII", 0x801, n, rows, cols) + px.tobytes())
    with pytest.raises(RuntimeError, match="InvalidMagicNumber"):
        ds.load_dataset(tmp_path / "bad", tmp_path / "lab")
    with pytest.raises(RuntimeError, match="InvalidMagicNumber"):
        ds.load_dataset(tmp_path / "img", tmp_path / "img")
    (tmp_path / "short").write_bytes(img_blob[:-5])
    with pytest.raises(RuntimeError, match="EndOfStream"):
        ds.load_dataset(tmp_path / "short", tmp_path / "lab")
    with pytest.raises(RuntimeError, match="cannot read"):
        ds.load_dataset(tmp_path / "absent", tmp_path / "lab")


def test_loader_feeds_the_loss_kernel(ds):
    """A gathered batch goes straight into the cross-entropy entry with byte targets, as examples/cnn.zig:141-142
    hands y_batch to the loss."""
    from znn_b200 import ops
    from znn_b200._lib import lib
    r = np.random.default_rng(6)
    n, dim, bs = 200, 10, 32
    logits_all = r.standard_normal((n, dim), np.float32)
    labels = r.integers(0, dim, n).astype(np.uint8)
    data = ds.Dataset.from_arrays(logits_all, labels)
    loader = ds.DataLoader(data, bs, shuffle=True, seed=3)
    order = loader.indices()[:bs]
    x_dev, y_dev = dev_buffers(bs, dim)
    assert loader.next_into(x_dev, y_dev) == bs
    probs, loss = ops.DevBuf(bs * dim * 4), ops.DevBuf(4)
    lib().call("znn_softmax_xent_fwd_u8", x_dev.ptr, y_dev.ptr, probs.ptr, loss.ptr, bs, dim)
    z = logits_all[order].astype(np.float64)
    lse = np.log(np.exp(z - z.max(1, keepdims=True)).sum(1)) + z.max(1)
    want = float(np.mean(lse - z[np.arange(bs), labels[order]]))
    assert abs(float(loss.to_host((1,))[0]) - want) <= 1e-5 * max(1.0, abs(want))


def test_training_fed_by_the_device_loader_equals_training_fed_from_host_batches(ds):
    """One epoch of the MLP example's loop (examples/fashion_mnist.zig:131-167) twice: batches copied from host
    arrays in the loader's order with int32 labels, and batches gathered on the device with the byte labels used in
    place.  Same parameters afterwards, bit for bit."""
    from oracle import models as omodels
    from znn_b200 import models
    r = np.random.default_rng(12)
    n, bs = 300, 64
    images = r.random((n, 784), np.float32)
    labels = r.integers(0, 10, n).astype(np.uint8)
    P0 = omodels.init_params("mlp", (784, 128, 64, 10), seed=1)

    def fresh(u8):
        m = models.Model("mlp", (784, 128, 64, 10), arena_bytes=64 << 20)
        m.set_params(P0)
        m.set_option("lr", 0.05)
        m.set_option("momentum", 0.9)
        m.set_option("cuda_graph", 0)
        m.set_option("targets_u8", u8)
        return m

    ref_loader = od.DataLoader(images, labels, bs, shuffle=True, seed=21, drop_last=True)
    host_fed = fresh(0)
    x, y = np.zeros((bs, 784), np.float32), np.zeros(bs, np.uint8)
    while ref_loader.next_into(x, y):
        host_fed.train_step(x, y.astype(np.int32))

    data = ds.Dataset.from_arrays(images, labels, rows=28, cols=28)
    loader = ds.DataLoader(data, bs, shuffle=True, seed=21, drop_last=True)
    dev_fed = fresh(1)
    x_dev, y_dev = dev_buffers(bs, 784)
    steps = 0
    while loader.next_into(x_dev, y_dev):
        dev_fed.train_step_device(x_dev.ptr, y_dev.ptr, bs)
        steps += 1
    assert steps == n // bs
    a, b = host_fed.get_params(), dev_fed.get_params()
    assert all(np.array_equal(a[k], b[k]) for k in a)


def test_evaluation_over_the_loader_matches_oracle(ds):
    """evaluateModel of the example programs (examples/cnn.zig:212-256): batches from the device loader (ragged last
    batch, no shuffling), loss and accuracy per batch on the device, averaged over batches as the reference does."""
    from oracle import models as omodels
    from znn_b200 import models
    r = np.random.default_rng(31)
    n, bs, dims = 150, 64, (784, 128, 64, 10)
    images = r.random((n, 784), np.float32)
    labels = r.integers(0, 10, n).astype(np.uint8)
    P0 = omodels.init_params("mlp", dims, seed=4)
    m = models.Model("mlp", dims, arena_bytes=64 << 20)
    m.set_params(P0)
    tr = omodels.OracleTrainer("mlp", P0, dims)
    data = ds.Dataset.from_arrays(images, labels, rows=28, cols=28)
    loader = ds.DataLoader(data, bs)
    x_dev, y_dev = dev_buffers(bs, 784)
    got, want, start = [], [], 0
    while True:
        k = loader.peek_next_batch_size()
        if k == 0:
            break
        assert loader.next_into(x_dev, y_dev) == k
        got.append(m.evaluate_device(x_dev.ptr, y_dev.ptr, k))
        loss, logits = tr.loss_and_grads(images[start:start + k], labels[start:start + k].astype(np.int32))
        want.append((loss, float(np.mean(np.argmax(logits, 1) == labels[start:start + k]))))
        start += k
    assert [k for k in (64, 64, 22)] and len(got) == 3
    for (lg, ag), (lo, ao) in zip(got, want):
        assert abs(lg - lo) <= 1e-5 * abs(lo)
        assert ag == np.float32(ao)
    # host arrays through the same entry
    lh, ah = m.evaluate(images[:64], labels[:64])
    assert (lh, ah) == got[0]
