"""The example programs' models run by the C++ host mirror (znn_model_*) against the CPU oracle's
composition of the same ops, on seeded synthetic inputs with the datasets' shapes and value ranges.

Bars: loss trajectory within 1e-4 relative at every step; argmax predictions bit-exact;
parameters after training within 1e-4 of their scale."""
import numpy as np
import pytest

from oracle import models

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def Model():
    from znn_b200 import ops
    from znn_b200.models import Model as M
    ops.init(0)
    return M


def pixels(r, n):
    return (r.integers(0, 256, (n, 784)).astype(np.float32) / np.float32(255.0)).astype(np.float32)


def relclose(a, b, tol, what, floor=0.0):
    """max |a-b| <= tol * max(|b|max, floor).  `floor` is the scale of the neighbouring tensors: some
    gradients are zero in exact arithmetic (a key bias shifts every score of a row alike, so softmax
    cancels it) and both sides then hold rounding noise only."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = max(1e-30, float(np.abs(b).max()), floor)
    err = float(np.abs(a - b).max())
    assert err <= tol * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


def grad_floor(grads):
    return max(float(np.abs(v).max()) for v in grads.values())


def run_training(Model, kind, dims, cfg, steps, batch, lr, momentum, seed, scheme="he", seq=0, vocab=10):
    r = np.random.default_rng(seed)
    P0 = models.init_params(kind, cfg, seed=seed + 1, scheme=scheme)
    m = Model(kind, dims, arena_bytes=512 << 20)
    m.set_params(P0)
    m.set_option("lr", lr)
    m.set_option("momentum", momentum)
    tr = models.OracleTrainer(kind, P0, cfg, lr=lr, momentum=momentum)
    worst = 0.0
    for s in range(steps):
        if kind == "gpt":
            x = r.integers(0, vocab, (batch, seq)).astype(np.float32)
            t = np.concatenate([x[:, 1:], r.integers(0, vocab, (batch, 1))], axis=1).astype(np.int32)
        else:
            x, t = pixels(r, batch), r.integers(0, 10, batch).astype(np.int32)
        lo, logits_o = tr.step(x, t)
        lg = m.train_step(x, t, seq=seq)
        rel = abs(lg - lo) / abs(lo)
        worst = max(worst, rel)
        assert rel <= 1e-4, f"{kind} step {s}: loss {lg} vs oracle {lo} (rel {rel:.2e})"
    Pg = m.get_params()
    floor = 1e-2 * grad_floor(tr.P)
    for k in tr.P:
        relclose(Pg[k], tr.P[k], 1e-4, f"{kind} {k} after {steps} steps", floor)
    return m, tr, worst


def test_mlp_100_steps_loss_trajectory(Model):
    """Config 1: 784->128->64->10 (examples/fashion_mnist.zig:25-27), batch 64, SGD momentum 0.9 lr 0.01."""
    m, tr, worst = run_training(Model, "mlp", (784, 128, 64, 10), (784, 128, 64, 10), 100, 64, 0.01, 0.9, seed=1234,
                                scheme="uniform")
    r = np.random.default_rng(99)
    x = pixels(r, 100)                                         # evaluation batch of 100 (fashion_mnist.zig:222-255)
    from oracle import ograph, zo
    g = ograph.OGraph()
    P = {k: g.array(v, False) for k, v in tr.P.items()}
    lo = models.mlp_net(g, P, g.array(x, False)).data
    lg = m.forward(x, classes=10)
    relclose(lg, lo, 1e-4, "eval logits")
    np.testing.assert_array_equal(np.argmax(lg, 1), zo.argmax(lo, 1).astype(np.int64))


def test_mlp_he_init_reference_schedule(Model):
    """The reference's own hyper-parameters: He-normal init, lr 0.05 (fashion_mnist.zig:98-101)."""
    run_training(Model, "mlp", (784, 128, 64, 10), (784, 128, 64, 10), 30, 64, 0.05, 0.9, seed=7, scheme="he")


def test_cnn_reference_shape(Model):
    """examples/cnn.zig: 1->4->8->16 valid convs, fc 144->10, batch 64."""
    run_training(Model, "cnn_ref", (), None, 12, 64, 0.05, 0.9, seed=11)


def test_cnn_padded_shape(Model):
    """Workload-definition CNN: 1->32->64 3x3 pad 1, 3136->128->10 (reduced batch for the CPU oracle)."""
    run_training(Model, "cnn_padded", (), None, 4, 16, 0.01, 0.9, seed=13, scheme="uniform")


def test_gpt_small_training(Model):
    """examples/transformer_gpt.zig architecture at a size the CPU oracle finishes: fused causal softmax in
    the C++ mirror against the reference's literal mulScalar/mask/add/softmax sequence in the oracle."""
    cfg = {"vocab_size": 61, "block_size": 24, "n_embd": 32, "n_head": 4, "n_layer": 2}
    dims = (61, 24, 32, 4, 2)
    m, tr, _ = run_training(Model, "gpt", dims, cfg, 15, 3, 0.05, 0.9, seed=21, seq=24, vocab=61)
    assert m.last_step_ops() > 50


def test_gpt_literal_attention_path(Model):
    """fused_softmax = 0 runs the reference's op sequence literally (materialised -1e9 mask)."""
    cfg = {"vocab_size": 29, "block_size": 8, "n_embd": 16, "n_head": 2, "n_layer": 1}
    r = np.random.default_rng(3)
    P0 = models.init_params("gpt", cfg, seed=4)
    x = r.integers(0, 29, (2, 8)).astype(np.float32)
    t = r.integers(0, 29, (2, 8)).astype(np.int32)
    losses = []
    for fused in (1, 0):
        m = Model("gpt", (29, 8, 16, 2, 1), arena_bytes=64 << 20)
        m.set_params(P0)
        m.set_option("fused_softmax", fused)
        m.set_option("fused_linear", 0)
        m.set_option("lr", 0.0)
        losses.append((m.train_step(x, t, seq=8), m.get_grads(), m.last_step_ops()))
    assert losses[1][2] == losses[0][2] + 2          # mulScalar, add, softmax instead of the one fused op
    assert abs(losses[0][0] - losses[1][0]) <= 1e-6 * abs(losses[1][0])
    # gradients that are zero in exact arithmetic (k_attn.bias) hold cancellation noise of ~1e-7 of the largest
    # gradient on both sides; the fused score gradient takes its row sums from dO.O instead of sum(dP o P), so the two
    # noises differ: 3 % of the largest gradient as the scale keeps the bar at 3e-7 of it
    floor = 3e-2 * grad_floor(losses[1][1])
    for k in losses[0][1]:
        relclose(losses[0][1][k], losses[1][1][k], 1e-5, k, floor)
    # the fused Linear op (matmul + addBias in one GEMM epilogue) against the two separate ops
    m = Model("gpt", (29, 8, 16, 2, 1), arena_bytes=64 << 20)
    m.set_params(P0)
    m.set_option("fused_linear", 1)
    m.set_option("lr", 0.0)
    lf = m.train_step(x, t, seq=8)
    Gf = m.get_grads()
    assert m.last_step_ops() < losses[0][2]
    assert abs(lf - losses[0][0]) <= 1e-6 * abs(lf)
    for k in Gf:
        relclose(Gf[k], losses[0][1][k], 1e-5, k, floor)


def test_transformer_block_config_shape_small(Model):
    """Pre-norm block forward+backward (examples/transformer_block.zig), d_model 64, 4 heads, batch 2 x seq 16."""
    from oracle import ograph
    r = np.random.default_rng(8)
    cfg = {"n_embd": 64}
    P0 = models.init_params("block", cfg, seed=9, scheme="n002")
    x = r.standard_normal((2, 16, 64), np.float32)
    dy = r.standard_normal((2, 16, 64), np.float32)
    m = Model("block", (64, 4), arena_bytes=64 << 20)
    m.set_params(P0)
    y, dx = m.block_fwd_bwd(x, dy)
    g = ograph.OGraph()
    P = {k: g.array(v, True) for k, v in P0.items()}
    xt = g.array(x, True)
    yo = models.transformer_block(g, P, "block", xt, n_head=4)
    yo.grad[...] = dy
    g.backwardWithGrad(yo)
    relclose(y, yo.data, 1e-5, "y")
    relclose(dx, xt.grad, 3e-5, "dx")
    G = m.get_grads()
    floor = 1e-2 * max(float(np.abs(t.grad).max()) for t in P.values())
    for k, tns in P.items():
        relclose(G[k], tns.grad.reshape(P0[k].shape), 3e-5, k, floor)


def test_greedy_decode_matches_oracle(Model):
    """examples/transformer_gpt.zig:116-146: full re-forward per token, first-maximum argmax; tokens bit-exact."""
    from oracle import ograph, zo
    cfg = {"vocab_size": 37, "block_size": 12, "n_embd": 16, "n_head": 2, "n_layer": 2}
    P0 = models.init_params("gpt", cfg, seed=31)
    r = np.random.default_rng(32)
    prompts = r.integers(0, 37, (3, 4)).astype(np.float32)
    m = Model("gpt", (37, 12, 16, 2, 2), arena_bytes=64 << 20)
    m.set_params(P0)
    got = m.greedy_decode(prompts, 14)                         # runs past block_size: the window slides
    seqs = [list(p) for p in prompts]
    for _ in range(14):
        T = min(len(seqs[0]), 12)
        win = np.array([s[-T:] for s in seqs], np.float32)
        g = ograph.OGraph()
        P = {k: g.array(v, False) for k, v in P0.items()}
        logits = models.gpt(g, P, g.array(win, False), cfg).data
        nxt = zo.argmax(np.ascontiguousarray(logits[:, -1, :]), 1)
        for s, n in zip(seqs, nxt):
            s.append(float(n))
    want = np.array([s[4:] for s in seqs], np.float32)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("kind,dims", [("mlp", (784, 128, 64, 10)), ("cnn_ref", ())])
def test_cuda_graph_replay_matches_eager(Model, kind, dims):
    """The captured-and-replayed training step must leave exactly the parameters the eager step leaves
    (same kernels, same order), step after step, with new data copied into the same device buffers."""
    from znn_b200 import ops
    r = np.random.default_rng(5)
    P0 = models.init_params(kind, dims if dims else None, seed=6)
    batches = [(pixels(r, 64), r.integers(0, 10, 64).astype(np.int32)) for _ in range(6)]
    finals, losses = [], []
    for use_graph in (0, 1):
        m = Model(kind, dims, arena_bytes=256 << 20)
        m.set_params(P0)
        m.set_option("lr", 0.05)
        m.set_option("momentum", 0.9)
        m.set_option("cuda_graph", use_graph)
        dx, dt = ops.DevBuf(64 * 784 * 4), ops.DevBuf(64 * 4)
        ls = []
        for x, t in batches:
            lib_ = ops.lib()
            lib_.call("znn_memcpy_h2d", dx.ptr, x.ctypes.data, x.nbytes)
            lib_.call("znn_memcpy_h2d", dt.ptr, t.ctypes.data, t.nbytes)
            lib_.call("znn_sync")
            import ctypes as C
            loss = C.c_float()
            lib_.call("znn_model_train_step", m.h, dx.ptr, dt.ptr, 64, 0, 1, C.byref(loss))
            ls.append(loss.value)
        if use_graph:
            assert m.graph_replays() == len(batches) - 1      # the first step runs eagerly, the rest replay
        finals.append(m.get_params())
        losses.append(ls)
        m.close()
    assert losses[0] == losses[1]
    for k in finals[0]:
        np.testing.assert_array_equal(finals[0][k], finals[1][k])


def test_gpt_causal_tile_skipping(Model):
    """At a context long enough for several 256-wide tiles the six attention products run on the tensor cores with
    triangular-structure hints (option causal_skip, default on): tiles above the causal diagonal are neither
    computed nor stored, contractions stop where the probabilities are exact zeros.  Loss and every gradient
    must equal the run without hints."""
    cfg = {"vocab_size": 128, "block_size": 768, "n_embd": 128, "n_head": 2, "n_layer": 1}
    dims = (128, 768, 128, 2, 1)
    r = np.random.default_rng(8)
    P0 = models.init_params("gpt", cfg, seed=9)
    x = r.integers(0, 128, (2, 768)).astype(np.float32)
    t = r.integers(0, 128, (2, 768)).astype(np.int32)
    res = []
    try:
        # hints on; hints off; and the reference's literal transposeND(K) + batchMatMul instead of the one Q.K^T op
        # the last variant is the single fused attention op (znn_attn_fwd / znn_attn_bwd), the default
        for skip, qkt, fsb, fa in ((1, 1, 1, 0), (0, 1, 1, 0), (0, 0, 0, 0), (1, 0, 0, 0), (1, 1, 0, 0), (1, 1, 1, 1)):
            m = Model("gpt", dims, arena_bytes=1 << 30)
            m.set_params(P0)
            m.set_option("fused_attention", fa)
            m.set_option("causal_skip", skip)
            m.set_option("fused_qkt", qkt)
            m.set_option("fused_softmax_bwd", fsb)
            m.set_option("lr", 0.0)
            res.append((m.train_step(x, t, seq=768), m.get_grads(), m.last_step_ops()))
    finally:
        m.set_option("fused_attention", 1)
        m.set_option("causal_skip", 1)
        m.set_option("fused_qkt", 1)
        m.set_option("fused_softmax_bwd", 1)
    floor = 3e-2 * grad_floor(res[2][1])   # see test_gpt_literal_attention_path: noise of exactly-zero gradients
    assert res[5][2] < res[0][2]          # the fused op replaces the transposes, products and softmax of the chain
    for i in (0, 1, 3, 4, 5):
        assert abs(res[i][0] - res[2][0]) <= 1e-6 * abs(res[2][0])
        for k in res[i][1]:
            relclose(res[i][1][k], res[2][1][k], 1e-5, k, floor)


def test_kv_cache_decode_gives_the_same_tokens(Model):
    """The key/value-cache decode (one pass per position) against the reference's full re-forward per token, both
    on the GPU and against the oracle's tokens; window not sliding (prompt + new - 1 <= block_size)."""
    cfg = {"vocab_size": 37, "block_size": 12, "n_embd": 16, "n_head": 2, "n_layer": 2}
    P0 = models.init_params("gpt", cfg, seed=31)
    r = np.random.default_rng(33)
    prompts = r.integers(0, 37, (5, 4)).astype(np.float32)
    m = Model("gpt", (37, 12, 16, 2, 2), arena_bytes=64 << 20)
    m.set_params(P0)
    full = m.greedy_decode(prompts, 9)
    kv = m.greedy_decode_kv(prompts, 9)
    np.testing.assert_array_equal(kv, full)
    with pytest.raises(RuntimeError):
        m.greedy_decode_kv(prompts, 10)           # would need the sliding window
    # a longer context on the tensor-core paths: d_model 128, 2 heads of 64, 40 positions
    cfg2 = {"vocab_size": 96, "block_size": 48, "n_embd": 128, "n_head": 2, "n_layer": 2}
    P1 = models.init_params("gpt", cfg2, seed=5)
    prompts2 = r.integers(0, 96, (8, 6)).astype(np.float32)
    m2 = Model("gpt", (96, 48, 128, 2, 2), arena_bytes=256 << 20)
    m2.set_params(P1)
    np.testing.assert_array_equal(m2.greedy_decode_kv(prompts2, 40), m2.greedy_decode(prompts2, 40))


def test_gpt_long_context_against_the_oracle(Model):
    """Context 512 with 64-wide heads: the attention products run on the tensor cores with the triangular hints, the
    one Q.K^T op, aliased reshape gradients and lazily zeroed gradients, all at their defaults, against the oracle's
    literal reference sequence (full products, materialised -1e9 mask, transposed copy of K, separate gradients)."""
    cfg = {"vocab_size": 96, "block_size": 512, "n_embd": 128, "n_head": 2, "n_layer": 1}
    run_training(Model, "gpt", (96, 512, 128, 2, 1), cfg, 3, 2, 0.05, 0.9, seed=41, seq=512, vocab=96)


def test_checkpoint_files_interchange_with_the_reference_layout(Model, tmp_path):
    """znn_model_save writes byte for byte what the reference's saveModel writes (src/nn.zig:268-303, restated in
    oracle/checkpoint.py) and znn_model_load reads such a file back, with the reference's checks."""
    from oracle import checkpoint
    cfg = {"vocab_size": 29, "block_size": 8, "n_embd": 16, "n_head": 2, "n_layer": 2}
    P0 = models.init_params("gpt", cfg, seed=2)
    m = Model("gpt", (29, 8, 16, 2, 2), arena_bytes=64 << 20)
    m.set_params(P0)
    ours, ref = tmp_path / "ours.safetensors", tmp_path / "ref.safetensors"
    m.save(ours)
    order = [(name, shape) for name, shape, _, _ in m.params]
    checkpoint.save(ref, [(name, np.asarray(P0[name], np.float32).reshape(shape)) for name, shape in order])
    assert ours.read_bytes() == ref.read_bytes()
    # a second model loads the reference-layout file
    P1 = models.init_params("gpt", cfg, seed=3)
    m2 = Model("gpt", (29, 8, 16, 2, 2), arena_bytes=64 << 20)
    m2.set_params(P1)
    m2.load(ref)
    got = m2.get_params()
    for name, shape in order:
        np.testing.assert_array_equal(got[name], np.asarray(P0[name], np.float32).reshape(shape))
    # wrong architecture: a shape check fails, as ShapeMismatch / TensorNotFound in the reference
    m3 = Model("gpt", (29, 8, 32, 2, 2), arena_bytes=64 << 20)
    with pytest.raises(RuntimeError):
        m3.load(ref)
    m4 = Model("gpt", (29, 8, 16, 2, 3), arena_bytes=64 << 20)
    with pytest.raises(RuntimeError):
        m4.load(ref)


def test_resume_from_model_and_optimizer_files_continues_bit_identically(Model, tmp_path):
    """Train 3 steps, save parameters and SGD velocities, train 3 more; a fresh model that loads both files and runs
    the same 3 steps ends with bit-identical parameters (the step is deterministic), and without the velocity file
    it does not (momentum 0.9 carries state)."""
    cfg = {"vocab_size": 29, "block_size": 8, "n_embd": 16, "n_head": 2, "n_layer": 2}
    dims = (29, 8, 16, 2, 2)
    r = np.random.default_rng(8)
    batches = [(r.integers(0, 29, (4, 8)).astype(np.float32), r.integers(0, 29, 32).astype(np.int32)) for _ in range(6)]

    def fresh(seed):
        m = Model("gpt", dims, arena_bytes=64 << 20)
        m.set_params(models.init_params("gpt", cfg, seed=seed))
        m.set_option("lr", 0.05)
        m.set_option("momentum", 0.9)
        return m

    m = fresh(2)
    for x, t in batches[:3]:
        m.train_step(x, t, seq=8)
    m.save(tmp_path / "model")
    m.save_optimizer(tmp_path / "optimizer")
    for x, t in batches[3:]:
        m.train_step(x, t, seq=8)
    want = m.get_params()

    resumed, cold = fresh(5), fresh(5)
    resumed.load(tmp_path / "model")
    resumed.load_optimizer(tmp_path / "optimizer")
    cold.load(tmp_path / "model")
    for x, t in batches[3:]:
        resumed.train_step(x, t, seq=8)
        cold.train_step(x, t, seq=8)
    got, got_cold = resumed.get_params(), cold.get_params()
    assert all(np.array_equal(got[k], want[k]) for k in want)
    assert any(not np.array_equal(got_cold[k], want[k]) for k in want)
    # the optimizer file has the model file's layout: same header, different payload
    a, b = (tmp_path / "model").read_bytes(), (tmp_path / "optimizer").read_bytes()
    hl = int.from_bytes(a[:8], "little")
    assert len(a) == len(b) and a[:8 + hl] == b[:8 + hl] and a[8 + hl:] != b[8 + hl:]


@pytest.mark.parametrize("kind,dims,cfg,seq,vocab", [
    ("mlp", (784, 128, 64, 10), (784, 128, 64, 10), 0, 10),
    ("gpt", (29, 8, 16, 2, 2), {"vocab_size": 29, "block_size": 8, "n_embd": 16, "n_head": 2, "n_layer": 2}, 8, 29),
])
def test_training_with_adam_matches_oracle(Model, kind, dims, cfg, seq, vocab):
    """AdamOptimizer (src/optim.zig:69-152) as the model's optimizer: loss trajectory and parameters against the
    oracle trainer running the restated step."""
    r = np.random.default_rng(17)
    P0 = models.init_params(kind, cfg, seed=3)
    m = Model(kind, dims, arena_bytes=256 << 20)
    m.set_params(P0)
    # Adam divides by sqrt(v): a gradient that is zero in exact arithmetic (the key bias of attention, which softmax
    # cancels) holds rounding noise on both sides and would be normalised into full-size steps of random sign with the
    # reference's default eps = 1e-8; the GPT case uses an eps above that noise and far below the real gradients
    eps = 1e-4 if kind == "gpt" else 1e-8
    for key, val in (("optimizer", 1), ("lr", 0.0005), ("beta1", 0.5), ("beta2", 0.999), ("eps", eps)):
        m.set_option(key, val)
    tr = models.OracleTrainer(kind, P0, cfg, lr=0.0005, adam=(0.5, 0.999, eps))
    batch = 16
    for s in range(20):
        if kind == "gpt":
            x = r.integers(0, vocab, (batch, seq)).astype(np.float32)
            t = r.integers(0, vocab, batch * seq).astype(np.int32)
        else:
            x, t = pixels(r, batch), r.integers(0, 10, batch).astype(np.int32)
        lo, _ = tr.step(x, t)
        lg = m.train_step(x, t, seq=seq)
        assert abs(lg - lo) <= 1e-4 * abs(lo), f"{kind} step {s}: loss {lg} vs oracle {lo}"
    Pg = m.get_params()
    for k in tr.P:
        relclose(Pg[k], tr.P[k], 2e-3, f"{kind} {k} after 20 Adam steps", floor=1e-2)
    with pytest.raises(RuntimeError):
        m.set_option("optimizer", 2)


def test_adam_resume_continues_bit_identically(Model, tmp_path):
    dims = (784, 128, 64, 10)
    r = np.random.default_rng(23)
    batches = [(pixels(r, 32), r.integers(0, 10, 32).astype(np.int32)) for _ in range(6)]

    def fresh(seed):
        m = Model("mlp", dims, arena_bytes=64 << 20)
        m.set_params(models.init_params("mlp", dims, seed=seed))
        m.set_option("optimizer", 1)
        m.set_option("lr", 0.001)
        return m

    m = fresh(2)
    for x, t in batches[:3]:
        m.train_step(x, t)
    m.save(tmp_path / "model")
    m.save_optimizer(tmp_path / "optimizer")
    for x, t in batches[3:]:
        m.train_step(x, t)
    want = m.get_params()
    resumed = fresh(9)
    resumed.load(tmp_path / "model")
    resumed.load_optimizer(tmp_path / "optimizer")
    resumed.set_option("adam_t", 3)
    for x, t in batches[3:]:
        resumed.train_step(x, t)
    got = resumed.get_params()
    assert all(np.array_equal(got[k], want[k]) for k in want)
    assert (tmp_path / "optimizer.v2").exists()


def _launches_of(lib_, fn):
    import ctypes as C
    n = C.c_longlong(0)
    lib_.call("znn_launch_count", C.byref(n), 1)
    out = fn()
    lib_.call("znn_launch_count", C.byref(n), 0)
    return out, n.value


def test_fused_epilogues_match_the_separate_ops(Model):
    """Option fused_epilogue (bit mask; 15 = every form): GELU / ReLU after a Linear, the residual adds of a transformer
    block and the activation derivative in backward run in GEMM epilogues (znn_linear_fwd_ex / znn_linear_bwd_ex).  The
    tape is the same; loss and every gradient must equal the separate kernels' to fp32 rounding, with fewer launches."""
    from znn_b200 import _lib
    L = _lib.lib()
    # GPT at a width that reaches the tensor-core path (the epilogue forms live there)
    cfg = {"vocab_size": 128, "block_size": 768, "n_embd": 128, "n_head": 2, "n_layer": 2}
    dims = (128, 768, 128, 2, 2)
    r = np.random.default_rng(18)
    P0 = models.init_params("gpt", cfg, seed=19)
    x = r.integers(0, 128, (2, 768)).astype(np.float32)
    t = r.integers(0, 128, (2, 768)).astype(np.int32)
    res = []
    try:
        for fe in (15, 0):
            m = Model("gpt", dims, arena_bytes=1 << 30)
            m.set_params(P0)
            m.set_option("fused_epilogue", fe)
            m.set_option("lr", 0.0)
            loss, launches = _launches_of(L, lambda: m.train_step(x, t, seq=768))
            res.append((loss, m.get_grads(), m.last_step_ops(), launches))
            m.close()
    finally:
        m2 = Model("mlp", (784, 128, 64, 10), arena_bytes=64 << 20)
        m2.set_option("fused_epilogue", 2)
        m2.close()
    assert res[0][2] <= res[1][2] + 2 * 2               # the same ops on the tape, plus two Reshape views of the residual per layer
    assert res[0][3] < res[1][3]                        # fewer launches (products that are split over K keep the separate ops)
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[1][0])
    floor = 3e-2 * grad_floor(res[1][1])
    for k in res[0][1]:
        relclose(res[0][1][k], res[1][1][k], 1e-5, k, floor)
    # MLP with ReLU at a batch whose first layer reaches the tensor-core path; the second layer falls back
    P1 = models.init_params("mlp", (784, 128, 64, 10), seed=23)
    xb, tb = pixels(r, 4096), r.integers(0, 10, 4096).astype(np.int32)
    out = []
    try:
        for fe in (15, 0):
            m = Model("mlp", (784, 128, 64, 10), arena_bytes=256 << 20)
            m.set_params(P1)
            m.set_option("fused_epilogue", fe)
            m.set_option("lr", 0.0)
            out.append((m.train_step(xb, tb), m.get_grads()))
            m.close()
    finally:
        m2 = Model("mlp", (784, 128, 64, 10), arena_bytes=64 << 20)
        m2.set_option("fused_epilogue", 2)
        m2.close()
    assert abs(out[0][0] - out[1][0]) <= 1e-6 * abs(out[1][0])
    for k in out[0][1]:
        relclose(out[0][1][k], out[1][1][k], 1e-5, k, 1e-2 * grad_floor(out[1][1]))


@pytest.mark.parametrize("dims,batch", [((61, 24, 32, 4, 2), 3), ((128, 256, 128, 2, 2), 4)])
def test_gpt_cuda_graph_replay_matches_eager(Model, dims, batch):
    """The GPT training step uploads nothing (position ids are written on the device), so it can be captured and
    replayed like the MLP / CNN steps: identical losses and parameters, step after step, with new token ids copied into
    the same device buffers.  The second size runs the fused attention kernels and the tensor-core GEMMs."""
    import ctypes as C
    from znn_b200 import ops
    V, T, D, H, NL = dims
    cfg = {"vocab_size": V, "block_size": T, "n_embd": D, "n_head": H, "n_layer": NL}
    r = np.random.default_rng(55)
    P0 = models.init_params("gpt", cfg, seed=56)
    batches = []
    for _ in range(5):
        x = r.integers(0, V, (batch, T)).astype(np.float32)
        t = np.concatenate([x[:, 1:], r.integers(0, V, (batch, 1))], axis=1).astype(np.int32)
        batches.append((x, t))
    finals, losses = [], []
    lib_ = ops.lib()
    for use_graph in (0, 1):
        m = Model("gpt", dims, arena_bytes=512 << 20)
        m.set_params(P0)
        m.set_option("lr", 0.05)
        m.set_option("momentum", 0.9)
        m.set_option("cuda_graph", use_graph)
        dx, dt = ops.DevBuf(batch * T * 4), ops.DevBuf(batch * T * 4)
        ls = []
        for x, t in batches:
            lib_.call("znn_memcpy_h2d", dx.ptr, x.ctypes.data, x.nbytes)
            lib_.call("znn_memcpy_h2d", dt.ptr, t.ctypes.data, t.nbytes)
            lib_.call("znn_sync")
            loss = C.c_float()
            lib_.call("znn_model_train_step", m.h, dx.ptr, dt.ptr, batch, T, 1, C.byref(loss))
            ls.append(loss.value)
        if use_graph:
            assert m.graph_replays() == len(batches) - 1
        finals.append(m.get_params())
        losses.append(ls)
        m.close()
    ops.check_device_status()
    assert losses[0] == losses[1]
    for k in finals[0]:
        np.testing.assert_array_equal(finals[0][k], finals[1][k])


@pytest.mark.parametrize("kind,batch", [("cnn_ref", 64), ("cnn_padded", 256)])
def test_cnn_fused_relu_forms_are_bit_identical(Model, kind, batch):
    """Relu stored by the convolution kernel itself (znn_conv2d_fwd_act) and Relu backward folded into MaxPool2D backward
    (znn_maxpool2d_bwd_relu): the same values as the separate kernels, bit for bit (loss, every gradient), fewer launches."""
    from znn_b200 import _lib
    L = _lib.lib()
    r = np.random.default_rng(71)
    P0 = models.init_params(kind, None, seed=72)
    x, t = pixels(r, batch), r.integers(0, 10, batch).astype(np.int32)
    out = []
    try:
        for fe in (2, 0):
            m = Model(kind, (), arena_bytes=2 << 30)
            m.set_params(P0)
            m.set_option("fused_epilogue", fe)
            m.set_option("lr", 0.0)
            loss, launches = _launches_of(L, lambda: m.train_step(x, t))
            out.append((loss, m.get_grads(), launches))
            m.close()
    finally:
        m2 = Model("mlp", (784, 128, 64, 10), arena_bytes=64 << 20)
        m2.set_option("fused_epilogue", 2)
        m2.close()
    assert out[0][0] == out[1][0]
    for k in out[0][1]:
        np.testing.assert_array_equal(out[0][1][k], out[1][1][k])
    assert out[0][2] < out[1][2]        # (products that are split over K keep their separate Relu: the same kernels)


def test_grouped_attention_projections_match_separate_launches(Model):
    """Option group_linear (default on): the q, k, v projections of an attention layer share their input and run as one
    grouped forward launch, one grouped weight-gradient launch and one K-concatenated data-gradient product
    (znn_sgemm_grouped).  Loss and every gradient must equal the three separate Linear layers' to fp32 rounding."""
    from znn_b200 import _lib
    L = _lib.lib()
    cfg = {"vocab_size": 128, "block_size": 768, "n_embd": 256, "n_head": 4, "n_layer": 2}
    dims = (128, 768, 256, 4, 2)
    r = np.random.default_rng(28)
    P0 = models.init_params("gpt", cfg, seed=29)
    x = r.integers(0, 128, (2, 768)).astype(np.float32)
    t = r.integers(0, 128, (2, 768)).astype(np.int32)
    res = []
    try:
        for grp in (1, 0):
            m = Model("gpt", dims, arena_bytes=2 << 30)
            m.set_params(P0)
            m.set_option("group_linear", grp)
            m.set_option("lr", 0.0)
            loss, launches = _launches_of(L, lambda: m.train_step(x, t, seq=768))
            res.append((loss, m.get_grads(), launches))
            m.close()
    finally:
        m2 = Model("mlp", (784, 128, 64, 10), arena_bytes=64 << 20)
        m2.set_option("group_linear", 1)
        m2.close()
    assert res[0][2] <= res[1][2] - 2 * 6          # per layer: 3 -> 1 forward, 3 -> 1 dW, 3 -> 1 dX launches
    assert abs(res[0][0] - res[1][0]) <= 1e-6 * abs(res[1][0])
    floor = 3e-2 * grad_floor(res[1][1])
    for k in res[0][1]:
        relclose(res[0][1][k], res[1][1][k], 1e-5, k, floor)
