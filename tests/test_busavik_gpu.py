"""The Busavik family on a B200 against the plain implementation, in float32 and bfloat16:
each new kernel alone (with inputs made so that a fault shows), then the engine on three small
models of other sizes: whole prompts, prompts against token-by-token decoding, portions down
to two tokens, unequal batches against each request alone, slots and pages used again, the
first tokens, long decoding across page borders, states after every layer run, and greedy
generation through the entry point."""
import numpy as np
import pytest
import torch

from mormot2_ai_b200 import Engine, Entry, LlmClient
from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.cache.pages import PAGE, pages_for
from mormot2_ai_b200.cache.storage import CacheLine
from tests.busavik_models import SMALL, SmallModel
from tests.conftest import close
from tests.gpu_helpers import DEV, make_step
from tests.plain import busavik_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module", params=sorted(SMALL))
def small(request, tmp_path_factory):
    return SmallModel(request.param, str(tmp_path_factory.mktemp("busavik_" + request.param)))


@pytest.fixture(scope="module")
def small_p(tmp_path_factory):
    return SmallModel("P", str(tmp_path_factory.mktemp("busavik_P_only")))


class Choices:
    """The experts that an engine's routers chose, by slot, layer run and position, read
    through the routed feed-forward's probe. In 16 bits a router may fall on the other side of
    a close call than the plain implementation; the plain one then takes the engine's choice
    THERE (``plain.Routing``), and a different choice anywhere else fails the test."""

    def __init__(self, eng):
        from mormot2_ai_b200.parts.moe import RoutedExperts
        layers = eng.model.layers
        self.runs = [i for i, r in enumerate(eng.model.spec.schedule)
                     if isinstance(layers[r.layer].feed_forward, RoutedExperts)]
        self.calls = 0
        self.by_slot = {}
        for layer in layers:
            if isinstance(layer.feed_forward, RoutedExperts):
                layer.feed_forward.probe = self.seen
        eng.use_graphs = False

    def seen(self, part, step, ids):
        run = self.runs[self.calls % len(self.runs)]      # routers run in the order of the runs
        self.calls += 1
        rows = ids.cpu().numpy()
        at = 0
        for slot, past, new in zip(step.host_slots, step.host_past, step.host_new):
            kept = self.by_slot.setdefault(slot, {})
            for j in range(new):
                kept[(run, past + j)] = rows[at + j].tolist()
            at += new

    def routing(self, slot):
        return plain.Routing(forced=self.by_slot.pop(slot, {}))


def engine_of(model, dtype, **kw):
    """An engine and, in bfloat16, the record of its routers' choices."""
    kw.setdefault("max_tokens", 2048)
    eng = Engine.from_folder(model.folder, dtype=dtype, **kw)
    eng.choices = Choices(eng) if dtype == "bfloat16" else None
    return eng


def expected(model, eng, slot, ids, states=None):
    """The plain logits of ``ids``, the routers settled as the engine's were at close calls."""
    routing = eng.choices.routing(slot) if eng.choices is not None else None
    return model.reference(ids, states, routing)


def check(got, want, dtype, what):
    ok, err = close(got, want, dtype)
    assert ok, f"{what}: relative error {err:.3g} ({dtype})"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(dtype).to(DEV)


def rounded(a, dtype):
    """What the device holds of ``a``: its values after rounding to the storage type."""
    return dev(a, TORCH[dtype]).float().cpu().numpy().astype(np.float64)


def latent_line(n_slots, max_len, width, dtype, seed=0):
    per = pages_for(max_len)
    n_pages = n_slots * per + 2
    ids = np.random.default_rng(seed).permutation(n_pages)[:n_slots * per]
    table = torch.tensor(ids.reshape(n_slots, per), dtype=torch.int32, device=DEV)
    pool = torch.zeros((n_pages, 1, PAGE, width), dtype=dtype, device=DEV)
    return CacheLine(pool, None, table, per, 0, 0, 1, width)


def write_rows(line, slot, rows, first=0):
    table = line.page_table.cpu()
    for i in range(rows.shape[0]):
        pos = first + i
        line.k[int(table[slot, pos // PAGE]), 0, pos % PAGE, :] = dev(rows[i], line.k.dtype)


def read_row(line, slot, pos):
    table = line.page_table.cpu()
    return line.k[int(table[slot, pos // PAGE]), 0, pos % PAGE, :].float().cpu().numpy()


# ---------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_kernel(dtype):
    rng = np.random.default_rng(1)
    T, H = 7, 50
    x = rng.normal(size=(T, H)) * 3
    w, b, alpha = rng.normal(size=H) + 1, rng.normal(size=H), 0.37
    xd = dev(x)
    out = torch.empty((T, H), dtype=TORCH[dtype], device=DEV)
    K.dynamic_tanh(xd, dev(w, TORCH[dtype]), dev(b, TORCH[dtype]), dev([alpha]), out)
    want = plain.dynamic_tanh(x, rounded(w, dtype), rounded(b, dtype), np.float32(alpha))
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(out.float().cpu().numpy() - want).max() < tol
    # gathered rows, and split sums that are first added into x
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty((3, H), dtype=TORCH[dtype], device=DEV)
    K.dynamic_tanh(xd, dev(w, TORCH[dtype]), dev(b, TORCH[dtype]), dev([alpha]), out, rows, 3)
    assert np.abs(out.float().cpu().numpy() - want[[5, 0, 5]]).max() < tol
    parts = rng.normal(size=(3, T, H))
    out = torch.empty((T, H), dtype=TORCH[dtype], device=DEV)
    K.dynamic_tanh(xd, dev(w, TORCH[dtype]), dev(b, TORCH[dtype]), dev([alpha]), out,
                   partial=dev(parts))
    assert np.abs(xd.cpu().numpy() - (x + parts.sum(0))).max() < 1e-5
    want = plain.dynamic_tanh(x + parts.sum(0), rounded(w, dtype), rounded(b, dtype), np.float32(alpha))
    assert np.abs(out.float().cpu().numpy() - want).max() < tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gated_activation_kernel(dtype, act):
    rng = np.random.default_rng(2)
    T, I, H = 5, 70, 22
    gu, bg, bu, bx = (rng.normal(size=s) for s in ((T, 2 * I), I, I, H))
    x = rng.normal(size=(T, H))
    t = TORCH[dtype]
    out = torch.empty((T, I), dtype=t, device=DEV)
    xd = dev(x)
    K.gated_act(dev(gu, t), out, K.ACTIVATIONS[act], dev(bg, t), dev(bu, t), xd, dev(bx, t))
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.silu
    g = rounded(gu, dtype)
    want = f(g[:, :I] + rounded(bg, dtype)) * (g[:, I:] + rounded(bu, dtype))
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert np.abs(out.float().cpu().numpy() - want).max() < tol * max(1, np.abs(want).max())
    assert np.abs(xd.cpu().numpy() - (x + rounded(bx, dtype))).max() < 1e-6
    out2 = torch.empty((T, I), dtype=t, device=DEV)
    K.gated_act(dev(gu, t), out2, K.ACTIVATIONS[act])
    want = f(g[:, :I]) * g[:, I:]
    assert np.abs(out2.float().cpu().numpy() - want).max() < tol * max(1, np.abs(want).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_prep_kernel_writes_normed_latents_and_the_rotated_part(dtype):
    rng = np.random.default_rng(3)
    qr, kvr, rd, dims = 11, 13, 10, 6
    rot = {"dims": dims, "base": 300.0,
           "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    freqs, amp = plain.yarn_frequencies(rot)
    t = TORCH[dtype]
    seqs = [(1, 60, list(range(9)), []), (0, 0, [1, 2], [])]        # across a page border
    step = make_step(seqs)
    T = 11
    line = latent_line(2, 128, kvr + rd, t, seed=4)
    f = rng.normal(size=(T, 5 + qr + kvr + rd + 3))                   # columns before and behind
    wq, wkv = rng.normal(size=qr) + 1, rng.normal(size=kvr) + 1
    cq = torch.empty((T, qr), dtype=t, device=DEV)
    K.latent_prep(dev(f, t), 5, 5 + qr, qr, kvr, rd, dev(wq, t), dev(wkv, t), 1e-5,
                  dev(freqs), dims, amp, step, line, cq, True)
    fr = rounded(f, dtype)
    want_q = plain.rms_norm(fr[:, 5:5 + qr], rounded(wq, dtype), 1e-5)
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert np.abs(cq.float().cpu().numpy() - want_q).max() < tol * np.abs(want_q).max()
    pos = np.array(list(range(60, 69)) + [0, 1])
    slot = [1] * 9 + [0] * 2
    want_c = plain.rms_norm(fr[:, 5 + qr:5 + qr + kvr], rounded(wkv, dtype), 1e-5)
    want_r = plain.rotate_half(fr[:, 5 + qr + kvr:5 + qr + kvr + rd], pos, freqs, amp)
    for i in range(T):
        got = read_row(line, slot[i], int(pos[i]))
        want = np.concatenate([want_c[i], want_r[i]])
        assert np.abs(got - want).max() < tol * np.abs(want).max(), i
    # the values behind the rotating ones pass as they are
    assert np.allclose(want_r[:, dims:], fr[:, 5 + qr + kvr + dims:5 + qr + kvr + rd])
    # the same rows given as three split sums (float32), with the columns behind them as a gate
    parts = rng.normal(size=(3,) + f.shape)
    parts[2] = fr - parts[0] - parts[1]
    line2 = latent_line(2, 128, kvr + rd, t, seed=4)
    cq2 = torch.empty((T, qr), dtype=t, device=DEV)
    gate = torch.empty((T, 3), dtype=t, device=DEV)
    K.latent_prep(None, 5, 5 + qr, qr, kvr, rd, dev(wq, t), dev(wkv, t), 1e-5, dev(freqs), dims,
                  amp, step, line2, cq2, True, partial=dev(parts), gate_out=gate,
                  gate_col=5 + qr + kvr + rd)
    assert np.abs(cq2.float().cpu().numpy() - want_q).max() < tol * np.abs(want_q).max()
    assert np.abs(gate.float().cpu().numpy() - fr[:, -3:]).max() < tol * np.abs(fr).max()
    for i in range(T):
        want = np.concatenate([want_c[i], want_r[i]])
        assert np.abs(read_row(line2, slot[i], int(pos[i])) - want).max() < tol * np.abs(want).max(), i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,Kd,tail", [(3, 10, 6), (70, 10, 6), (150, 40, 8), (3, 64, 8),
                                       (13, 96, 16)])
def test_heads_gemm_kernel(dtype, M, Kd, tail):
    """The last three cases have rows on 16-byte boundaries and go to the tensor cores in
    bfloat16: 128-row tiles, and for at most 16 tokens the form that reads weights into
    registers."""
    rng = np.random.default_rng(4)
    H, N, dims = 3, 21, 4
    t = TORCH[dtype]
    a = rng.normal(size=(M, H, Kd + tail))
    b = rng.normal(size=(H, N, Kd))
    freqs = np.array([0.5, 0.01])
    pos = rng.integers(0, 500, M)
    c = torch.zeros((M, H * (N + tail)), dtype=t, device=DEV)
    K.heads_gemm(dev(a.reshape(M, -1), t), Kd + tail, dev(b, t), c, N + tail, tail=tail,
                 rot_dims=dims, inv_freq=dev(freqs), amplitude=1.3,
                 tok_pos=torch.tensor(pos, dtype=torch.int32, device=DEV))
    ar, br = rounded(a, dtype), rounded(b, dtype)
    want = np.concatenate([np.einsum("mhk,hnk->mhn", ar[..., :Kd], br),
                           plain.rotate_half(ar[..., Kd:], pos, freqs, 1.3)], axis=-1)
    tol = 1e-5 if dtype == "float32" else 2e-2
    got = c.float().cpu().numpy().reshape(M, H, N + tail)
    assert np.abs(got - want).max() < tol * np.abs(want).max()
    # the gated form: no tail, the product times the sigmoid of the gate's columns
    gate = rng.normal(size=(M, 4 + H * N))
    c2 = torch.zeros((M, H * N), dtype=t, device=DEV)
    K.heads_gemm(dev(a.reshape(M, -1), t), Kd + tail, dev(b, t), c2, N, gate=dev(gate, t)[:, 4:])
    want = (np.einsum("mhk,hnk->mhn", ar[..., :Kd], br).reshape(M, H * N)
            * plain.sigmoid(rounded(gate, dtype)[:, 4:]))
    assert np.abs(c2.float().cpu().numpy() - want).max() < tol * np.abs(want).max()


def plain_latent_attention(q, rows, kvr, scale, lo=0):
    s = q @ rows[lo:].T * scale
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    return p @ rows[lo:, :kvr]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(5, 24, 8), (3, 13, 6), (6, 160, 32)])
def test_latent_attention_kernel_random_rows(dtype, sizes):
    nh, kvr, rd = sizes
    rng = np.random.default_rng(5)
    t = TORCH[dtype]
    past, new = 130, 5
    line = latent_line(2, 256, kvr + rd, t, seed=6)
    rows = rng.normal(size=(past + new, kvr + rd))
    write_rows(line, 1, rows)
    rr = rounded(rows, dtype)
    q = rng.normal(size=(new, nh, kvr + rd))
    step = make_step([(1, past, [0] * new, [])])
    out = torch.empty((new, nh * kvr), dtype=t, device=DEV)
    K.latent_attention(dev(q.reshape(new, -1), t), out, step, line, nh, kvr, rd, 0, 0.2)
    got = out.float().cpu().numpy().reshape(new, nh, kvr)
    tol = 1e-5 if dtype == "float32" else 2e-2
    for i in range(new):
        want = plain_latent_attention(rounded(q[i], dtype), rr[:past + i + 1], kvr, 0.2)
        assert np.abs(got[i] - want).max() < tol * max(1.0, np.abs(want).max()), i


@pytest.mark.parametrize("sizes", [(5, 32, 16), (16, 64, 32), (3, 160, 32), (70, 48, 16)])
def test_latent_attention_tensor_core_kernel(sizes):
    """The tensor-core kernel: two prompts' portions behind unequal pasts in one step (rows of
    several tokens and heads in one block, tiles of keys across page borders), then single
    tokens with a sequence's key tiles dealt out over 1, 3 and 16 blocks."""
    nh, kvr, rd = sizes
    rng = np.random.default_rng(11)
    t = torch.bfloat16
    line = latent_line(3, 512, kvr + rd, t, seed=12)
    pasts, news = [130, 0, 61], [37, 70, 5]
    rows = [rng.normal(size=(p + n, kvr + rd)) for p, n in zip(pasts, news)]
    for slot, r in enumerate(rows):
        write_rows(line, slot, r)
    q = [rng.normal(size=(n, nh, kvr + rd)) for n in news]
    step = make_step([(slot, pasts[slot], [0] * news[slot], []) for slot in range(3)])
    T = sum(news)
    out = torch.empty((T, nh * kvr), dtype=t, device=DEV)
    K.latent_attention_mma(dev(np.concatenate(q).reshape(T, -1), t), out, step, line, nh, kvr, rd,
                           0, 0.2, 1, None)
    got = out.float().cpu().numpy().reshape(T, nh, kvr)
    at = 0
    for slot in range(3):
        rr = rounded(rows[slot], "bfloat16")
        for i in range(news[slot]):
            want = plain_latent_attention(rounded(q[slot][i], "bfloat16"),
                                          rr[:pasts[slot] + i + 1], kvr, 0.2)
            assert np.abs(got[at] - want).max() < 2e-2 * max(1.0, np.abs(want).max()), (slot, i)
            at += 1
    # decode: one token of every sequence, the keys of a sequence over several blocks
    lens = [p + n for p, n in zip(pasts, news)]
    step = make_step([(slot, lens[slot] - 1, [0], []) for slot in range(3)])
    qd = rng.normal(size=(3, nh, kvr + rd))
    scratch = torch.empty((3 * nh * 16 * (kvr + 2),), dtype=torch.float32, device=DEV)
    tickets = torch.zeros((8,), dtype=torch.int32, device=DEV)
    for splits in (1, 3, 16, 3):
        out = torch.full((3, nh * kvr), 7.0, dtype=t, device=DEV)
        K.latent_attention_mma(dev(qd.reshape(3, -1), t), out, step, line, nh, kvr, rd, 0, 0.2,
                               splits, scratch, tickets)
        assert int(tickets.abs().sum()) == 0         # the counters are left as they were found
        got = out.float().cpu().numpy().reshape(3, nh, kvr)
        for slot in range(3):
            want = plain_latent_attention(rounded(qd[slot], "bfloat16"),
                                          rounded(rows[slot], "bfloat16"), kvr, 0.2)
            assert np.abs(got[slot] - want).max() < 2e-2 * max(1.0, np.abs(want).max()), (splits, slot)


def test_the_runtime_sends_sizes_it_takes_to_the_tensor_cores():
    from mormot2_ai_b200.engine.runtime import Runtime
    rt = Runtime(torch.bfloat16)
    calls = []
    real = K.latent_attention_mma
    K.latent_attention_mma = lambda *a, **k: (calls.append(a[9]), real(*a, **k))
    try:
        for (kvr, rd), fast in (((32, 16), True), ((40, 12), False)):
            line = latent_line(1, 2048, kvr + rd, torch.bfloat16)
            step = make_step([(0, 100, [0], [])])
            q = torch.zeros((1, 4 * (kvr + rd)), dtype=torch.bfloat16, device=DEV)
            out = torch.empty((1, 4 * kvr), dtype=torch.bfloat16, device=DEV)
            calls.clear()
            rt.latent_attention(q, out, step, line, 4, kvr, rd, 0, 1.0)
            assert bool(calls) == fast
            if fast:
                assert calls[0] == 16          # one sequence, 148 SMs: the most splits
    finally:
        K.latent_attention_mma = real
    rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("past", [63, 64, 700])
def test_latent_attention_finds_one_far_key_and_no_later_one(dtype, past):
    """One key far back (the very first, one at a page border, one in the middle) is made to
    take all of a head's weight: the output must be that row's latent. A key that would take
    all the weight but lies AFTER the query's position must not be seen."""
    nh, kvr, rd = 2, 16, 16
    t = TORCH[dtype]
    rng = np.random.default_rng(7)
    line = latent_line(1, 1024, kvr + rd, t, seed=8)
    n = past + 3
    rows = rng.normal(size=(n, kvr + rd)) * 0.1
    rows[:, :kvr] *= 10                            # latents that differ clearly from row to row
    for target in (0, 64 * (past // 64) - 1 if past >= 64 else 1, past // 2, past):
        rows2 = rows.copy()
        rows2[target, kvr:] = 0
        rows2[target, kvr] = 30.0                 # stands out in the rotated part
        rows2[past + 1, kvr + 1] = 30.0            # a later key, louder on another dimension
        write_rows(line, 0, rows2)
        q = np.zeros((1, nh, kvr + rd))
        q[0, :, kvr] = 1.0
        q[0, :, kvr + 1] = 2.0
        step = make_step([(0, past, [0], [])])     # the query stands at position `past`
        want = rounded(rows2[target, :kvr], dtype)
        for kernel in ["simt"] + (["mma 1", "mma 5"] if dtype == "bfloat16" else []):
            out = torch.empty((1, nh * kvr), dtype=t, device=DEV)
            if kernel == "simt":
                K.latent_attention(dev(q.reshape(1, -1), t), out, step, line, nh, kvr, rd, 0, 1.0)
            else:
                splits = int(kernel.split()[1])
                scratch = torch.empty((nh * splits * (kvr + 2),), dtype=torch.float32, device=DEV)
                K.latent_attention_mma(dev(q.reshape(1, -1), t), out, step, line, nh, kvr, rd, 0,
                                       1.0, splits, scratch,
                                       torch.zeros((4,), dtype=torch.int32, device=DEV))
            got = out.float().cpu().numpy().reshape(nh, kvr)
            assert np.abs(got - want).max() < 2e-2, (target, past, kernel)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_window_edges(dtype):
    """With a window the key just inside it is seen and the one just outside is not."""
    nh, kvr, rd, window, past = 1, 16, 16, 70, 200
    t = TORCH[dtype]
    line = latent_line(1, 256, kvr + rd, t, seed=9)
    rng = np.random.default_rng(9)
    base = rng.normal(size=(past + 1, kvr + rd)) * 0.1
    base[:, :kvr] *= 10
    inside, outside = past + 1 - window, past - window
    for loud, seen in ((inside, True), (outside, False)):
        rows = base.copy()
        rows[loud, kvr] = 30.0
        write_rows(line, 0, rows)
        q = np.zeros((1, kvr + rd))
        q[0, kvr] = 1.0
        step = make_step([(0, past, [0], [])])
        for kernel in ["simt"] + (["mma"] if dtype == "bfloat16" else []):
            out = torch.empty((1, kvr), dtype=t, device=DEV)
            if kernel == "simt":
                K.latent_attention(dev(q, t), out, step, line, nh, kvr, rd, window, 1.0)
            else:
                K.latent_attention_mma(dev(q, t), out, step, line, nh, kvr, rd, window, 1.0, 1, None)
            got = out.float().cpu().numpy()[0]
            if seen:
                assert np.abs(got - rounded(rows[loud, :kvr], dtype)).max() < 2e-2, kernel
            else:
                want = plain_latent_attention(rounded(q, dtype), rounded(rows, dtype), kvr, 1.0,
                                              lo=inside)[0]
                assert np.abs(got - want).max() < 2e-2, kernel


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,E,top,shared,ff,H", [
    (3, 5, 1, 0, 14, 24), (9, 6, 3, 20, 14, 24), (150, 4, 2, 12, 14, 24),
    (150, 4, 2, 16, 40, 24),        # bfloat16: 128-row tiles on the tensor cores
    (5, 7, 3, 8, 16, 24),           # the same with few rows an expert
    (5, 7, 3, 32, 32, 64),          # bfloat16: the decode form (at most 8 tokens, sizes % 32)
    (8, 3, 2, 0, 96, 160)])         # the same with every expert chosen by several tokens
def test_routed_experts_part(dtype, T, E, top, shared, ff, H):
    """The whole routed feed-forward (router, lists, both products, the sum) against the plain
    one; the router's rows are scaled so that no choice is a close call."""
    from mormot2_ai_b200.config.spec import PartSpec
    from mormot2_ai_b200.engine.runtime import Runtime
    from mormot2_ai_b200.parts import FEED_FORWARDS
    rng = np.random.default_rng(10 + T)
    t = TORCH[dtype]
    names = {"router": "router", "expert": "e{}.", "shared": "shared.",
             "shared_gate": "shared.sg", "gate": "gate", "up": "up", "down": "down"}
    part = FEED_FORWARDS.build(PartSpec("routed_experts", {
        "hidden_size": H, "experts": E, "top": top, "intermediate_size": ff,
        "shared_size": shared, "activation": "silu", "names": names}), "m.")
    W = {n.name: rng.normal(size=n.shape) * (2.0 if n.name == "m.router" else 0.3)
         for n in part.tensors()}
    rt = Runtime(t)
    part.bind({k: dev(v, t) for k, v in W.items()}, rt)
    h = rng.normal(size=(T, H))
    x0 = rng.normal(size=(T, H))
    x = dev(x0)
    part.forward(dev(h, t), x, None)
    Wr = {k[2:]: rounded(v, dtype) for k, v in W.items()}
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = x0 + plain.moe_ff(rounded(h, dtype), mlp, Wr, "")
    # leave out tokens whose choice is a close call in the storage type
    z = rounded(h, dtype) @ Wr["router"].T
    zs = np.sort(z, axis=1)[:, ::-1]
    sure = (zs[:, top - 1] - zs[:, top]) > 0.05 if top < E else np.ones(T, bool)
    assert sure.sum() >= T * 0.7
    tol = 1e-5 if dtype == "float32" else 3e-2
    got = x.cpu().numpy()
    assert np.abs(got[sure] - want[sure]).max() < tol * np.abs(want).max()
    rt.check()


def test_router_kernel_ties_and_weights():
    z = torch.tensor([[0.1, 2.0, 2.0, -1.0, 9.0], [3.0, 1.0, 0.0, 3.5, -2.0]], device=DEV)
    ids = torch.empty((2, 2), dtype=torch.int32, device=DEV)
    w = torch.empty((2, 2), dtype=torch.float32, device=DEV)
    sg = torch.empty((2,), dtype=torch.float32, device=DEV)
    want = np.exp([0.0, -0.5]) / np.exp([0.0, -0.5]).sum()

    def check_choice():
        assert ids.cpu().tolist() == [[1, 2], [3, 0]]         # the lower index on a tie
        assert np.allclose(w.cpu().numpy(), [[0.5, 0.5], want], atol=1e-6)
        assert np.allclose(sg.cpu().numpy(), plain.sigmoid(np.array([9.0, -2.0])), atol=1e-6)

    K.moe_route(z, 4, 2, 4, ids, w, sg)                       # column 4 is the shared gate's
    check_choice()
    # the logits as two split sums (exact in float32), and choice and lists in one kernel
    halves = torch.stack([z * 0.25, z * 0.75]).contiguous()
    ids.zero_(), w.zero_(), sg.zero_()
    K.moe_route(halves, 4, 2, 4, ids, w, sg)
    check_choice()
    ids.zero_(), w.zero_(), sg.zero_()
    max_tiles = 1 + 4
    plan = torch.full((2 + 4 + 4 + 2 * max_tiles,), -7, dtype=torch.int32, device=DEV)
    K.moe_route_plan(halves, 4, 2, 4, ids, w, sg, 8, max_tiles, plan)
    check_choice()
    got = plan.cpu().tolist()
    assert got[0] == 4                                        # experts 0, 1, 2, 3: a tile each
    assert got[1:6] == [0, 1, 2, 3, 4]                        # where each expert's list begins
    assert sorted(got[6:10]) == [0, 1, 2, 3] and got[6:10][0] == 3    # expert 0 was chosen by a = 3


# ---------------------------------------------------------------------------- the engine
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_states_after_every_layer_run(small, dtype):
    eng = engine_of(small, dtype)
    for n in small.prompt_lens:
        ids = small.tokens(n, seed=n)
        states = []
        eng.on_state = lambda name, x: states.append((name, x.cpu().numpy().copy()))
        slot = eng.open()
        out = eng.step([Entry(slot, ids, list(range(n)))])
        eng.on_state = None
        eng.close(slot)
        want_states = []
        want = expected(small, eng, slot, ids, want_states)
        check(out.cpu().numpy(), want, dtype, f"{small.name}: whole prompt of {n}")
        runs = [x for name, x in states if name.startswith("run")]
        assert len(runs) == len(want_states) == len(small.config.order())
        for i, (got, ref) in enumerate(zip(runs, want_states)):
            tol = 1e-5 if dtype == "float32" else 4e-2
            assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()), (n, i)
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_decoding(small, dtype):
    """The last tokens one by one through the cache, across a page border, and a sequence that
    is decoded from its second token on."""
    eng = engine_of(small, dtype)
    for n, head in ((75, 58), (12, 1), (140, 126)):
        ids = small.tokens(n, seed=100 + n)
        slot = eng.open()
        got = [eng.step([Entry(slot, ids[:head], [head - 1])]).cpu().numpy()]
        for t in range(head, n):
            got.append(eng.step([Entry(slot, [ids[t]])]).cpu().numpy().copy())
        assert eng.length(slot) == n
        eng.close(slot)
        ref = expected(small, eng, slot, ids)
        for k, row in enumerate(got):
            t = head - 1 + k
            check(row, ref[t:t + 1], dtype, f"token {t} of {n} (prompt of {head})")
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [2, 7, 64])
def test_portions_of_prompts(small, dtype, chunk):
    """Prompts cut into passes of a few tokens give the logits of the whole prompt; the
    portions of several steps (3, 2, 61 and 65 tokens) do too."""
    eng = engine_of(small, dtype, prefill_chunk=chunk)
    n = 131
    ids = small.tokens(n, seed=500 + chunk)
    slot = eng.open()
    want = [0, 1, 62, 63, 64, 65, n - 1]
    out = eng.step([Entry(slot, ids, want)]).cpu().numpy()
    eng.close(slot)
    check(out, expected(small, eng, slot, ids)[want], dtype, f"{n} tokens in passes of {chunk}")
    slot = eng.open()
    got = [eng.step([Entry(slot, ids[a:b], list(range(b - a)))]).cpu().numpy()
           for a, b in ((0, 3), (3, 5), (5, 66), (66, n))]
    eng.close(slot)
    check(np.concatenate(got), expected(small, eng, slot, ids), dtype,
          "steps of 3, 2, 61 and 65 tokens")
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_against_each_alone_with_reuse(small, dtype):
    """Batches of unequal requests, one after another in three slots and just enough pages:
    every logit equals that of the request's own whole pass (the plain one), whoever shares
    the batch; slots and pages are given back and used again."""
    lens = small.prompt_lens + [2, 65, 33]
    decode = [small.decode_steps, 3, 1, small.decode_steps, 5, 2, 4][:len(lens)]
    lens = lens[:len(decode)]
    pages = max(sum(-(-(n + d) // 64) for n, d in list(zip(lens, decode))[b0:b0 + 3])
                for b0 in range(0, len(lens), 3))
    eng = engine_of(small, dtype, max_tokens=64 * pages, max_slots=3)
    reqs = [small.tokens(n + d, seed=200 + i) for i, (n, d) in enumerate(zip(lens, decode))]
    for b0 in range(0, len(reqs), 3):
        idx = list(range(b0, min(b0 + 3, len(reqs))))
        slots = {i: eng.open() for i in idx}
        mine = dict(slots)
        assert sorted(slots.values()) == list(range(len(idx)))          # the same slots again
        got = {i: {} for i in idx}
        out = eng.step([Entry(slots[i], reqs[i][:lens[i]]) for i in idx]).cpu().numpy()
        for row, i in enumerate(idx):
            got[i][lens[i] - 1] = out[row:row + 1]
        at = {i: lens[i] for i in idx}
        live = list(idx)
        while live:
            live = [i for i in live if at[i] < len(reqs[i])]
            for i in idx:
                if i not in live and i in slots:
                    eng.close(slots.pop(i))       # ended earlier: slot and pages go back
            if not live:
                break
            out = eng.step([Entry(slots[i], [reqs[i][at[i]]]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                got[i][at[i]] = out[row:row + 1].copy()
                at[i] += 1
        for i in idx:
            ref = expected(small, eng, mine[i], reqs[i])
            for t, row in got[i].items():
                check(row, ref[t:t + 1], dtype, f"request {i} token {t}")
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    assert eng.book.slots.free == 3
    assert eng.faults() == []
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_mates_do_not_matter(small_p, dtype):
    """The same request alone and beside others, in a prompt step and in decode steps: equal
    logits up to rounding."""
    small = small_p
    eng = Engine.from_folder(small.folder, dtype=dtype, max_tokens=2048)
    a = small.tokens(70, seed=1)
    others = [small.tokens(n, seed=2 + n) for n in (3, 129)]
    s = eng.open()
    alone = [eng.step([Entry(s, a[:66], [0, 64, 65])]).cpu().numpy()]
    alone += [eng.step([Entry(s, [t])]).cpu().numpy().copy() for t in a[66:]]
    eng.close(s)
    slots = [eng.open() for _ in range(3)]
    out = eng.step([Entry(slots[0], others[0], []), Entry(slots[1], a[:66], [0, 64, 65]),
                    Entry(slots[2], others[1], [])]).cpu().numpy()
    tol = 1e-5 if dtype == "float32" else 3e-2
    scale = np.abs(alone[0]).max()
    assert np.abs(out - alone[0]).max() <= tol * scale
    for k, t in enumerate(a[66:]):
        out = eng.step([Entry(slots[0], [5]), Entry(slots[1], [t]), Entry(slots[2], [7])])
        assert np.abs(out.cpu().numpy()[1:2] - alone[1 + k]).max() <= tol * scale
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(small_p, dtype):
    small = small_p
    eng = engine_of(small, dtype, max_tokens=512)
    n = 200                                  # three page borders, token by token
    ids = small.tokens(n, seed=300)
    slot = eng.open()
    got = [eng.step([Entry(slot, [t])]).cpu().numpy().copy() for t in ids]
    eng.close(slot)
    ref = expected(small, eng, slot, ids)
    for t, row in enumerate(got):
        ok, err = close(row, ref[t:t + 1], dtype)
        assert ok, f"token {t}: relative error {err:.3g}"
    eng.rt.check()


def test_decode_graphs_replay_what_was_computed(small_p):
    """Decode passes are captured as CUDA graphs (routing happens on the device, nothing is
    read back): replayed steps give what the same steps give without graphs, to the bit, and
    in float32 what the plain implementation gives."""
    small = small_p
    ids = [small.tokens(40 + 3 * i, seed=600 + i) for i in range(2)]
    for dtype in DTYPES:
        outs = {}
        for graphs in (True, False):
            eng = Engine.from_folder(small.folder, dtype=dtype, max_tokens=1024)
            assert eng.use_graphs
            eng.use_graphs = graphs
            slots = [eng.open() for _ in ids]
            eng.step([Entry(s, r[:30], []) for s, r in zip(slots, ids)])
            outs[graphs] = [eng.step([Entry(s, [r[t]]) for s, r in zip(slots, ids)]).cpu().numpy().copy()
                            for t in range(30, 40)]
            assert len(eng.graphs) == (1 if graphs else 0)
            eng.rt.check()
        for a, b in zip(outs[True], outs[False]):
            assert np.array_equal(a, b)
        if dtype == "float32":
            for row, r in enumerate(ids):
                ref = small.reference(r)
                for k, t in enumerate(range(30, 40)):
                    check(outs[True][k][row:row + 1], ref[t:t + 1], dtype, f"step {t}, row {row}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(small, dtype):
    client = LlmClient(small.folder, dtype=dtype, max_batch=3, cache_tokens=1024)
    prompts = [small.tokens(n, seed=800 + n) for n in (4, 70, 17, 1)]
    steps = small.decode_steps
    got = client.generate(prompts, max_tokens=steps, temperature=0.0, stop=[])
    for p, tokens in zip(prompts, got):
        assert len(tokens) == steps
        ids = list(p)
        for i, a in enumerate(tokens):
            routing = plain.Routing()
            logits = small.reference(ids, routing=routing)[-1]
            if dtype == "bfloat16" and min(routing.margins.values(), default=1.0) < routing.close:
                break          # a router's close call: 16 bits may take the other side from here on
            order = np.argsort(-logits, kind="stable")
            if a != int(order[0]):
                # another token is right only at a near tie of the plain logits
                margin = float(logits[order[0]] - logits[order[1]])
                assert dtype == "bfloat16" and margin < 0.06 * logits.std(), (i, a, margin)
                break
            ids.append(a)
    assert all(client.engine.book.held_pages(g) == 0 for g in range(len(client.engine.plans)))
