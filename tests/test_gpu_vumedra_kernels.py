"""The kernels behind the Vumedra design, each alone against the plain restatement's function of the same mechanism,
with inputs made so that a fault shows: one key whose score stands out far back among hundreds, at a page's border
and at the query itself; scores so low that only the sink is left; the token before a step's first; a convolution
state shorter than its reach; a matrix memory whose input gate outgrows the running maximum."""
import numpy as np
import pytest
import torch

import plain_vumedra as plain

from esp_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def dev(t, dtype=None):
    return t.to(DEV, dtype if dtype is not None else t.dtype).contiguous()


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def paged(rows, table, n_pages, dtype):
    """rows [T, G, W] of one sequence -> pool [n_pages, G, PAGE, W] with position p in page table[p // PAGE]."""
    T, G, W = rows.shape
    pool = torch.zeros(n_pages, G, PAGE, W, dtype=dtype)
    for p in range(T):
        pool[table[p // PAGE], :, p % PAGE] = rows[p].to(dtype)
    return pool


# ------------------------------------------------------------------------------------------------ attention
def run_attention(kernel, q, k_pool, v_pool, out, table, first, new, H, G, K, V, scale, status):
    """The new tokens are positions first .. first + new - 1 of one sequence whose pages ``table`` lists."""
    args = (q, k_pool, v_pool, out)
    tables = i32([table])
    if kernel == "tensor16":              # mma.sync, tiles of 64 rows
        firsts = list(range(0, new, 64))
        ops.attn_prefill(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K, None,
                         status, vd=V, scale=scale, sink=True)
    elif kernel == "tmem16":              # tcgen05, tiles of 128 rows
        firsts = list(range(0, new, ops.ATTN_TC05_TILE_ROWS))
        ops.attn_prefill_tc05(*args, i32([0] * len(firsts)), i32(firsts), i32([0, new]), i32([first]), tables, PAGE, H, G, K,
                              None, status, scale=scale, sink=True)
    elif kernel == "split16":             # keys split over blocks, for few rows
        split = 128
        n_splits = (len(table) * PAGE + split - 1) // split
        part_o = torch.zeros(new, H, n_splits, K, device=DEV)
        part_ml = torch.zeros(new, H, n_splits, 2, device=DEV)
        counters = torch.zeros(ops.ATTN_DECODE_COUNTERS, dtype=torch.int32, device=DEV)
        ops.attn_decode(*args, part_o, part_ml, counters, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G,
                        K, None, split, n_splits, status, scale=scale, sink=True)
        assert int(counters.abs().sum().item()) == 0
    else:
        ops.attn_simt(*args, i32([0] * new), i32(list(range(first, first + new))), tables, PAGE, H, G, K, None, status, vd=V,
                      scale=scale, sink=True)


def takes(kernel, K, V):
    return kernel in ("plain32", "plain16", "tensor16") or (K == V and K in (64, 128))


@pytest.mark.parametrize("kernel", ["plain32", "plain16", "tensor16", "tmem16", "split16"])
@pytest.mark.parametrize("H, G, K, V", [(4, 2, 16, 40), (3, 1, 56, 88), (1, 1, 24, 8), (2, 2, 128, 128), (8, 2, 64, 64)])
def test_attention_finds_one_key_wherever_it_lies(kernel, H, G, K, V):
    """700 cached positions in pages handed out in no order; the new tokens are the last 70.  For every probed place
    (far back, both sides of page borders, the query itself, the first position) one key gets a large score for
    one query head, so that head's output must be that position's value row."""
    if not takes(kernel, K, V):
        pytest.skip("this kernel wants keys and values of one size, 64 or 128")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    g = torch.Generator().manual_seed(5)
    T, new = 700, 70
    q = torch.randn(new, H, K, generator=g) * 0.3
    k = torch.randn(T, G, K, generator=g) * 0.3
    v = torch.randn(T, G, V, generator=g)
    probes = [(0, 3), (5, 63), (11, 64), (20, 127), (33, 128), (40, 0), (47, T - new + 47), (69, T - 1), (60, 640 - 1)]
    for row, key in probes:
        head = row % H
        direction = torch.randn(K, generator=g)
        direction /= direction.norm()
        k[key, head // (H // G)] = direction * 6
        q[row, head] = direction * 6
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    scale = 0.9
    pos = torch.arange(T)
    want = plain.attend_with_sink(q, k, v, scale, pos[T - new:], pos)
    for row, key in probes:       # the oracle itself sees the designed key
        assert torch.allclose(want[row, row % H], v[key, (row % H) // (H // G)], atol=2e-2)
    n_pages = 16
    table = [7, 2, 11, 0, 5, 13, 1, 9, 3, 15, 4]
    out = torch.zeros(new, H * V, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    run_attention(kernel, dev(q.reshape(new, H * K), dtype), dev(paged(k, table, n_pages, dtype)),
                  dev(paged(v, table, n_pages, dtype)), out, table, T - new, new, H, G, K, V, scale, status)
    assert int(status.item()) == 0
    err = (out.double().cpu().view(new, H, V) - want).abs().max().item()
    assert err < (1e-5 if dtype == torch.float32 else 5e-2), err


@pytest.mark.parametrize("K, V", [(32, 16), (64, 64)])
@pytest.mark.parametrize("kernel", ["plain32", "tensor16", "tmem16", "split16"])
def test_the_sink_takes_the_weight_that_no_key_earns(kernel, K, V):
    """Scores far below zero: with the extra term in the denominator the output is nearly nothing, without it the
    plain average of the values; scores far above zero: the sink does not matter."""
    if not takes(kernel, K, V):
        pytest.skip("this kernel wants keys and values of one size, 64 or 128")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    H, T = 2, 120 if kernel == "split16" else 130
    g = torch.Generator().manual_seed(8)
    direction = torch.randn(K, generator=g)
    direction /= direction.norm()
    q = (direction * 4).repeat(T, H, 1)
    q[:, 1] *= -1                                    # head 0: every score is -16 * scale; head 1: +16 * scale
    k = (-direction * 4).repeat(T, 1, 1)
    v = torch.randn(T, 1, V, generator=g) * 0.3 + 3.0
    q, k, v = (t.to(dtype).double() for t in (q, k, v))
    pos = torch.arange(T)
    want = plain.attend_with_sink(q, k, v, 1.0, pos, pos)
    without = plain.attend_with_sink(q, k, v, 1.0, pos, pos, sink=False)
    assert want[:, 0].abs().max() < 1e-3 and (without[:, 0] - want[:, 0]).abs().min() > 1.0
    table = [2, 0, 1]
    out = torch.zeros(T, H * V, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    run_attention(kernel, dev(q.reshape(T, H * K), dtype), dev(paged(k, table, 3, dtype)), dev(paged(v, table, 3, dtype)), out,
                  table, 0, T, H, 1, K, V, 1.0, status)
    assert int(status.item()) == 0
    got = out.double().cpu().view(T, H, V)
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_and_key_norms_temperature_and_cache_write(dtype):
    H, G, K, V, eps = 3, 1, 20, 12, 1e-5
    g = torch.Generator().manual_seed(3)
    positions = [0, 5, 6, 63, 64, 13, 14, 200]       # two sequences' tokens; temperature steps every 7 positions
    seqs = [0, 0, 0, 0, 0, 1, 1, 1]
    n = len(positions)
    qkv = torch.randn(n, (H + G) * K + G * V, generator=g)
    bias = torch.randn(qkv.shape[1], generator=g) * 0.5
    qw, kw = torch.rand(K, generator=g) + 0.5, torch.rand(K, generator=g) + 0.5
    coef, every = 0.7, 7
    x = (qkv + bias).double()
    q = plain.rms(x[:, :H * K].view(n, H, K), eps) * qw.double()
    factor = torch.tensor([1 + coef * np.log((p + 1) // every + 1) for p in positions], dtype=torch.float64)
    q = q * factor[:, None, None]
    k = plain.rms(x[:, H * K:(H + G) * K].view(n, G, K), eps) * kw.double()
    v = x[:, (H + G) * K:].view(n, G, V)
    tables = [[3, 1, 0, 2], [5, 4, 6, 7]]
    q_out = torch.zeros(n, H * K, dtype=dtype, device=DEV)
    k_pool = torch.zeros(8, G, PAGE, K, dtype=dtype, device=DEV)
    v_pool = torch.zeros(8, G, PAGE, V, dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qknorm_kvwrite(dev(qkv), dev(bias), dev(qw), dev(kw), eps, coef, every, i32(seqs), i32(positions), q_out, k_pool, v_pool,
                       i32(tables), PAGE, H, G, K, V, True, status)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (q_out.double().cpu().view(n, H, K) - q).abs().max() < tol * 4
    for i, (s, p) in enumerate(zip(seqs, positions)):
        page = tables[s][p // PAGE]
        assert (k_pool[page, :, p % PAGE].double().cpu() - k[i]).abs().max() < tol * 4
        assert (v_pool[page, :, p % PAGE].double().cpu() - v[i]).abs().max() < tol * 4
    assert int((k_pool != 0).any(-1).sum().item()) == n * G        # nothing else was written


# ------------------------------------------------------------------------------------------------ embeddings, norms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_summed_embeddings_and_the_token_before(dtype):
    cfg = {"width": 50, "vocab": 300, "embedding": {"bigram": {"buckets": 37, "mul_prev": 1000003, "mul_cur": 7919}}}
    g = torch.Generator().manual_seed(2)
    w = {"embed": torch.randn(300, 50, generator=g).to(dtype), "bigram": torch.randn(38, 50, generator=g).to(dtype)}
    freq = torch.tensor(np.power(10000.0, -2.0 * np.arange(25) / 50), dtype=torch.float32)
    state = torch.zeros(6, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    seq_a, seq_b = [5, 299, 0, 17, 17, 120], [44, 3, 250]
    # step 1: a's first four tokens and b's first; step 2: a's last two, b's last two (slots 4 and 1)
    steps = [([(4, seq_a[:4], 0), (1, seq_b[:1], 0)]), ([(4, seq_a[4:], 4), (1, seq_b[1:], 1)])]
    got = {4: [], 1: []}
    for entries in steps:
        ids = [t for _, toks, _ in entries for t in toks]
        tok_seq = [i for i, (_, toks, _) in enumerate(entries) for _ in toks]
        tok_pos = [first + j for _, toks, first in entries for j in range(len(toks))]
        starts = np.cumsum([0] + [len(toks) for _, toks, _ in entries]).tolist()
        x = torch.zeros(len(ids), 50, device=DEV)
        ops.embed_sum(dev(w["embed"]), dev(w["bigram"]), dev(freq), i32(ids), i32(tok_seq), i32(tok_pos), i32(starts),
                      i32([s for s, _, _ in entries]), state, x, status, buckets=37, mul_prev=1000003, mul_cur=7919)
        for i, (slot, toks, _) in enumerate(entries):
            got[slot].append(x[starts[i]:starts[i + 1]].cpu())
    for slot, toks in ((4, seq_a), (1, seq_b)):
        want = plain.embedding(toks, {k: v.double() for k, v in w.items()}, cfg, torch.float64)
        assert (torch.cat(got[slot]).double() - want).abs().max() < 2e-5
    assert state.tolist() == [0, seq_b[-1] + 1, 0, 0, seq_a[-1] + 1, 0]
    assert int(status.item()) == 0


def test_norm_of_a_result_add_and_next_norm_in_one_launch():
    g = torch.Generator().manual_seed(4)
    n, width, eps = 9, 100, 1e-5
    x, y = torch.randn(n, width, generator=g) * 3, torch.randn(n, width, generator=g) * 40
    gy, gx = torch.full((width,), 0.8), torch.full((width,), 1.3)
    new_x = x.double() + plain.scalar_norm(y.double(), torch.tensor(0.8, dtype=torch.float64), eps)
    want_h = plain.scalar_norm(new_x, torch.tensor(1.3, dtype=torch.float64), eps)
    xd = dev(x)
    h = torch.zeros(n, width, dtype=torch.bfloat16, device=DEV)
    h32 = torch.zeros(n, width, device=DEV)
    ops.norm_add_rmsnorm(xd, dev(y), dev(gy), eps, dev(gx), h, eps, h32=h32)
    assert (xd.double().cpu() - new_x).abs().max() < 1e-5 and (h32.double().cpu() - want_h).abs().max() < 1e-5
    assert (h.double().cpu() - want_h).abs().max() < 2e-2
    # selected rows, x left alone
    xd2 = dev(x)
    rows = i32([7, 2])
    h2 = torch.zeros(2, width, device=DEV)
    ops.norm_add_rmsnorm(xd2, dev(y), dev(gy), eps, dev(gx), h2, eps, rows=rows, write_x=False)
    assert torch.equal(xd2.cpu(), x) and (h2.double().cpu() - want_h[[7, 2]]).abs().max() < 1e-5
    # the normed result alone
    alone = torch.zeros(n, width, device=DEV)
    ops.norm_add_rmsnorm(None, dev(y), dev(gy), eps, None, None, 0.0, h32=alone)
    assert (alone.double().cpu() - plain.scalar_norm(y.double(), torch.tensor(0.8, dtype=torch.float64), eps)).abs().max() < 1e-5


def test_squared_relu_with_a_factor_per_row():
    g = torch.Generator().manual_seed(6)
    z = torch.randn(7, 24, generator=g)
    scale = torch.rand(7, generator=g)
    act = torch.zeros(7, 24, device=DEV)
    ops.relu2(dev(z), act, row_scale=dev(scale))
    assert torch.allclose(act.cpu(), torch.relu(z * scale[:, None]) ** 2, atol=1e-6)


# ------------------------------------------------------------------------------------------------ recurrences
def test_matrix_memory_gates_follow_the_running_maximum():
    """Input gates that jump far above and forget gates that fall far below what came before, over two runs of one
    sequence and a second sequence in another slot: decay, input weight and m against the chain written out, and the
    value rows with their weight and the column of the normaliser."""
    g = torch.Generator().manual_seed(9)
    H, V, cap = 2, 4, 7.0
    cols = 8
    runs = [[5, 3], [2, 4]]                              # step 1: 5 tokens of sequence a, 3 of b; step 2: 2 and 4
    ld = H * V + 2 * H
    bias = torch.randn(2, H, generator=g)
    m_state = torch.zeros(4, H, device=DEV)
    total = {0: [], 1: []}
    outs = {0: [], 1: []}
    for run in runs:
        n = sum(run)
        proj = torch.randn(n, ld, generator=g)
        proj[:, -2 * H:] *= 6                            # raw gates far out, so that the cap and the maximum both act
        pd = dev(proj)
        starts = np.cumsum([0] + run).tolist()
        v, gi, gf = pd[:, :H * V], pd[:, H * V:H * V + H], pd[:, H * V + H:]
        vo, ktm = torch.zeros(n, H * cols, device=DEV), torch.zeros(3, n, H, device=DEV)
        ops.matrix_memory_prepare(v, gi, gf, ld, dev(bias[0]), dev(bias[1]), cap, m_state[1:], i32(starts), i32([2, 0]), vo, ktm,
                                  2, H, V, cols)
        for s in (0, 1):
            sl = slice(starts[s], starts[s + 1])
            total[s].append(proj[sl])
            outs[s].append((vo[sl].cpu(), ktm[0, sl].cpu(), ktm[1, sl].cpu(), ktm[2, sl].cpu()))
    for s in (0, 1):
        proj = torch.cat(total[s]).double()
        vo, keep_o, take_o, mo = (torch.cat([o[i] for o in outs[s]]).double() for i in range(4))
        gi = cap * torch.tanh((proj[:, -2 * H:-H] + bias[0].double()) / cap)
        gf = plain.logsigmoid(cap * torch.tanh((proj[:, -H:] + bias[1].double()) / cap))
        m = torch.zeros(H, dtype=torch.float64)
        for t in range(proj.shape[0]):
            m_new = torch.maximum(gf[t] + m, gi[t])
            keep, take = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
            m = m_new
            assert torch.allclose(mo[t], m, atol=1e-5) and torch.allclose(keep_o[t], keep, atol=1e-5)
            assert torch.allclose(take_o[t], take, atol=1e-5)
            vr = vo[t].view(H, cols)
            assert torch.allclose(vr[:, :V], take[:, None] * proj[t, :H * V].view(H, V), atol=1e-5)
            assert torch.allclose(vr[:, V], take, atol=1e-5) and float(vr[:, V + 1:].abs().max()) == 0
    assert torch.allclose(m_state[3].cpu().double(), torch.cat([o[3] for o in outs[0]])[-1].double(), atol=1e-6)
    assert float(m_state[0].abs().max()) == 0 and float(m_state[2].abs().max()) == 0


def test_recurrence_with_one_decay_per_head_and_the_normalised_readout():
    """The shared recurrence with a ready-made decay per head and token, from a state left by an earlier call, and
    what follows it: quotient by max(|n . q|, exp(-m)), unit root mean square per head, weight and sigmoid gate."""
    g = torch.Generator().manual_seed(10)
    H, K, V, cols, n = 3, 24, 6, 8, 21
    q, k = torch.randn(n, H * K, generator=g), torch.randn(n, H * K, generator=g)
    v = torch.zeros(n, H, cols)
    v[:, :, :V] = torch.randn(n, H, V, generator=g)
    v[:, :, V] = 1.0
    take = torch.rand(n, H, generator=g) + 0.2
    v = v * take[:, :, None]
    keep = torch.rand(n, H, generator=g)
    m = torch.randn(n, H, generator=g)
    state = torch.zeros(3, H * cols * K, device=DEV)
    out = []
    for a, b in ((0, 8), (8, 21)):                      # two calls: the second goes on from the first's state
        o = torch.zeros(b - a, H * cols, device=DEV)
        ops.gated_scan(ops.SCAN_SCALAR_DECAY, dev(q[a:b]), dev(k[a:b]), dev(keep[a:b]), dev(v[a:b].reshape(b - a, -1)), None, None,
                       None, state, i32([0, b - a]), i32([1]), o, 1, H, K, cols, ready=True)
        out.append(o)
    o = torch.cat(out)
    S = torch.zeros(H, K, cols, dtype=torch.float64)
    want = torch.zeros(n, H, cols, dtype=torch.float64)
    for t in range(n):
        S = keep[t].double()[:, None, None] * S + k[t].double().view(H, K)[:, :, None] * v[t].double()[:, None, :]
        want[t] = torch.einsum("hkc,hk->hc", S, q[t].double().view(H, K))
    assert (o.double().cpu().view(n, H, cols) - want).abs().max() < 1e-4
    assert float(state[[0, 2]].abs().max()) == 0
    w, gate, qs, eps = torch.rand(H * V, generator=g) + 0.5, torch.randn(n, H * V, generator=g), K ** -0.5, 1e-5
    y = torch.zeros(n, H * V, device=DEV)
    ops.matrix_memory_finish(o, dev(m), dev(w), dev(gate), y, H, V, cols, eps, 1e-6, q_scale=qs)
    den = torch.maximum((want[:, :, V] * qs).abs(), torch.exp(-m.double())) + 1e-6
    val = plain.rms(want[:, :, :V] * qs / den[:, :, None], eps).reshape(n, H * V) * w.double() * torch.sigmoid(gate.double())
    assert (y.double().cpu() - val).abs().max() < 1e-4


def test_convolution_state_shorter_than_its_reach_and_the_diagonal_recurrence():
    """Five taps, runs of 1, 2, 1, 6 and 3 tokens: the first runs leave fewer inputs than the convolution reaches
    back, so its state is shifted and the oldest entries stay zeros; against the plain function on the whole
    sequence.  A second sequence in another slot runs beside it."""
    g = torch.Generator().manual_seed(12)
    C, B, taps, width = 24, 3, 5, 16
    cb = C // B
    w = {"y": torch.randn(C, width, generator=g) * 0.3, "y.b": torch.randn(C, generator=g) * 0.3,
         "x": torch.randn(C, width, generator=g) * 0.3, "x.b": torch.randn(C, generator=g) * 0.3,
         "conv": torch.randn(C, taps, generator=g) * 0.5, "conv.b": torch.randn(C, generator=g) * 0.2,
         "ra": torch.randn(B, cb, cb, generator=g), "ra.b": torch.randn(B, cb, generator=g),
         "ri": torch.randn(B, cb, cb, generator=g), "ri.b": torch.randn(B, cb, generator=g),
         "lam": torch.randn(C, generator=g) * 1.5 - 1, "o": torch.eye(C)}
    wd = {k: v.double() for k, v in w.items()}
    seqs = {0: torch.randn(13, width, generator=g), 1: torch.randn(13, width, generator=g)}
    want = {s: plain.rglru(h.double(), wd, "", {"width": C, "blocks": B}) for s, h in seqs.items()}
    state = torch.zeros(5, taps * C, device=DEV)
    slots = {0: 3, 1: 1}
    w_gates = torch.cat([w["ra"], w["ri"]], 1).contiguous()
    got = {0: [], 1: []}
    at = 0
    for run in (1, 2, 1, 6, 3):
        h = torch.cat([seqs[0][at:at + run], seqs[1][at:at + run]])
        n = 2 * run
        proj = dev(torch.cat([h @ w["y"].T, h @ w["x"].T], 1))
        gate, u32, u_act = (torch.zeros(n, C, device=DEV) for _ in range(3))
        starts, tok_seq = i32([0, run, n]), i32([0] * run + [1] * run)
        seq_slot = i32([slots[0], slots[1]])
        ops.conv_branches(proj, dev(w["y.b"]), dev(w["x.b"]), dev(w["conv"]), dev(w["conv.b"]), state[:, C:], tok_seq, starts,
                          seq_slot, gate, u32, u_act, 2, C, taps)
        gates = torch.zeros(n, 2 * C, device=DEV)
        ops.per_head_linear(u_act, C, cb, dev(w_gates), gates, 2 * C, 2 * cb, n, B, cb, 2 * cb)
        out = torch.zeros(n, C, device=DEV)
        ops.diag_scan(gates, dev(w["ra.b"].reshape(-1)), dev(w["ri.b"].reshape(-1)), dev(w["lam"]), 8.0, u32, gate, state, starts,
                      seq_slot, out, 2, C, B)
        got[0].append(out[:run].cpu())
        got[1].append(out[run:].cpu())
        at += run
    for s in (0, 1):
        assert (torch.cat(got[s]).double() - want[s]).abs().max() < 2e-5
    assert float(state[[0, 2, 4]].abs().max()) == 0
