"""Every kernel of the recurrent layers and of the latent attention alone, against float64 arithmetic written
here, at sizes the model tests do not have, with inputs made so that a lost key, a window that is one position off
or a state that is not carried shows."""
import math

import numpy as np
import pytest
import torch

import plain_zusepel as plain

from esp_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------- the recurrence
def scan_reference(mode, q, k, g, v, bias, lower, bonus, S):
    """One sequence; q, k, g [T, H, K], v [T, H, V], S [H, K, V] (float64).  Returns (out [T, H, V], S)."""
    out = []
    for t in range(q.shape[0]):
        if mode == ops.SCAN_DECAY_BONUS:
            d = torch.exp(-torch.exp(g[t] + bias))
            kv = k[t][:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hkv,hk->hv", S + bonus[:, :, None] * kv, q[t]))
            S = d[:, :, None] * S + kv
        else:
            d = lower + (1 - lower) * torch.sigmoid(g[t] + bias)
            S = d[:, :, None] * S + (1 - d)[:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hkv,hk->hv", S, torch.nn.functional.silu(q[t])))
    return torch.stack(out), S


@pytest.mark.parametrize("mode", [ops.SCAN_DECAY_BONUS, ops.SCAN_LOWER_SIGMOID])
@pytest.mark.parametrize("H,K,V", [(3, 24, 40), (1, 128, 72), (2, 16, 16), (5, 64, 130), (2, 100, 8), (1, 200, 24), (2, 256, 7)])
def test_gated_scan_runs_cuts_and_slots(mode, H, K, V):
    torch.manual_seed(H * 1000 + K + V + mode)
    runs = [37, 1, 20]                       # three sequences of unequal length in one call
    slots = [5, 0, 3]
    N = sum(runs)
    # q, g, v are columns of one wider matrix, as a packed projection leaves them
    packed = torch.randn(N, 2 * H * K + H * V + 8, device=DEV)
    q, g, v = packed[:, :H * K], packed[:, H * K:2 * H * K], packed[:, 2 * H * K:2 * H * K + H * V]
    k = torch.randn(N, H * K, device=DEV)
    bias = torch.randn(H * K, device=DEV) - 1.0
    lower = torch.rand(H * K, device=DEV) * 0.9
    bonus = torch.randn(H * K, device=DEV)
    words = H * K * V
    state0 = torch.randn(7, words + 11, device=DEV) * 0.3      # rows wider than the state: the stride is honoured
    starts = np.concatenate([[0], np.cumsum(runs)])

    def run(state, cuts):
        """cuts: per call, the number of rows each sequence brings."""
        out = torch.zeros(N, H * V, device=DEV)
        done = [0, 0, 0]
        for cut in cuts:
            rows = [list(range(starts[b] + done[b], starts[b] + done[b] + cut[b])) for b in range(3)]
            live = [b for b in range(3) if cut[b] > 0]
            idx = torch.tensor(sum((rows[b] for b in live), []), device=DEV)
            o = torch.zeros(len(idx), H * V, device=DEV)
            sub = packed[idx].contiguous()
            ops.gated_scan(mode, sub[:, :H * K], k[idx].contiguous() if mode == ops.SCAN_DECAY_BONUS else None,
                           sub[:, H * K:2 * H * K], sub[:, 2 * H * K:2 * H * K + H * V], bias, lower if mode else None,
                           bonus if not mode else None, state, i32(np.concatenate([[0], np.cumsum([cut[b] for b in live])])),
                           i32([slots[b] for b in live]), o, len(live), H, K, V)
            out[idx] = o
            for b in range(3):
                done[b] += cut[b]
        return out

    s_whole = state0.clone()
    whole = run(s_whole, [runs])
    s_cut = state0.clone()
    cut = run(s_cut, [[30, 1, 2], [1, 0, 1], [6, 0, 17]])
    assert torch.equal(whole, cut) and torch.equal(s_whole, s_cut)         # cutting changes no bit
    assert torch.equal(s_whole[[1, 2, 4, 6]], state0[[1, 2, 4, 6]])         # other slots untouched
    assert torch.equal(s_whole[:, words:], state0[:, words:])              # nor the rest of a row
    for b in range(3):
        sl = slice(starts[b], starts[b + 1])
        T = runs[b]
        S0 = state0[slots[b], :words].double().cpu().view(H, V, K).transpose(1, 2)     # stored [V][K]
        ref, S1 = scan_reference(mode, q[sl].double().cpu().view(T, H, K), k[sl].double().cpu().view(T, H, K),
                                 g[sl].double().cpu().view(T, H, K), v[sl].double().cpu().view(T, H, V),
                                 bias.double().cpu().view(H, K), lower.double().cpu().view(H, K),
                                 bonus.double().cpu().view(H, K), S0)
        scale = float(ref.abs().max())
        assert float((whole[sl].double().cpu().view(T, H, V) - ref).abs().max()) <= 2e-5 * scale
        got_S = s_whole[slots[b], :words].double().cpu().view(H, V, K).transpose(1, 2)
        assert float((got_S - S1).abs().max()) <= 2e-5 * max(1.0, float(S1.abs().max()))


def test_gated_scan_keeps_a_distant_token():
    """With decays of one a value written 500 tokens ago is read back exactly; with decays of zero nothing older
    than the current token is."""
    H, K, V, T = 1, 16, 16, 501
    q = torch.zeros(T, K, device=DEV)
    k = torch.zeros(T, K, device=DEV)
    v = torch.zeros(T, V, device=DEV)
    k[0, 3] = 1.0
    v[0] = torch.arange(V, device=DEV).float()
    q[T - 1, 3] = 2.0
    for raw, expect in ((-1e4, 2.0), (1e4, 0.0)):          # exp(-exp(raw)): one, zero
        state = torch.zeros(1, H * K * V, device=DEV)
        out = torch.zeros(T, V, device=DEV)
        ops.gated_scan(ops.SCAN_DECAY_BONUS, q, k, torch.full((T, K), raw, device=DEV), v, None, None,
                       torch.zeros(K, device=DEV), state, i32([0, T]), i32([0]), out, 1, H, K, V)
        assert torch.equal(out[T - 1], expect * v[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift(dtype):
    torch.manual_seed(1)
    D, runs, slots = 72, [4, 1, 3], [2, 0, 1]
    N = sum(runs)
    h = torch.randn(N, D, device=DEV).to(dtype)
    state = torch.randn(3, 40 + D, device=DEV)
    prev_state = state[:, 40:]
    mu = torch.rand(5, D, device=DEV)
    out = torch.empty(5, N, D, device=DEV, dtype=dtype)
    seq = i32(np.repeat(np.arange(3), runs))
    starts = i32(np.concatenate([[0], np.cumsum(runs)]))
    before = state.clone()
    ops.token_shift_mix(h, prev_state, seq, starts, i32(slots), mu, out)
    ops.token_shift_keep(h, prev_state, starts, i32(slots), 3)
    hf = h.double()
    at = 0
    for b, n in enumerate(runs):
        prev = torch.cat([before[slots[b], 40:].double()[None], hf[at:at + n - 1]], 0)
        want = hf[at:at + n][None] + (prev - hf[at:at + n])[None] * mu.double()[:, None, :]
        tol = 1e-6 if dtype == torch.float32 else 2 ** -7
        assert float((out[:, at:at + n].double() - want).abs().max()) <= tol * float(want.abs().max())
        assert torch.equal(state[slots[b], 40:], h[at + n - 1].float())
        at += n
    assert torch.equal(state[:, :40], before[:, :40])


@pytest.mark.parametrize("shared", [True, False])
def test_head_norm_and_gate(shared):
    torch.manual_seed(2)
    N, H, V = 9, 3, 40
    o = torch.randn(N, H * V, device=DEV) * 3
    w = torch.randn(V if shared else H * V, device=DEV)
    gate = torch.randn(N, H * V + 5, device=DEV)[:, :H * V]
    y = torch.empty(N, H * V, device=DEV)
    ops.head_rmsnorm_gate(o, w, 0 if shared else V, None if shared else gate, y, H, V, 1e-3)
    od = o.double().view(N, H, V)
    want = od / torch.sqrt((od ** 2).mean(-1, keepdim=True) + 1e-3) * (w.double().view(1, 1, V) if shared else w.double().view(1, H, V))
    if not shared:
        want = want * torch.nn.functional.silu(gate.double().view(N, H, V))
    assert float((y.double().view(N, H, V) - want).abs().max()) <= 1e-5 * float(want.abs().max())


# ---------------------------------------------------------------------------------------------- latent attention
ROT = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}}


def freqs(rot):
    from esp_b200.config.plan import ScaledRopeSpec
    from esp_b200.parts import Runtime
    from esp_b200.parts.position import RopeScaled
    sc = rot["scaling"]
    f, mag = RopeScaled(ScaledRopeSpec(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"]),
                        Runtime(None, torch.float32)).frequencies()
    return torch.from_numpy(f).to(DEV), mag


@pytest.mark.parametrize("rot_dim", [16, 24])
def test_cache_rows_and_query_rotation(rot_dim):
    """rot_dim 24 with 16 rotated dimensions: the last 8 pass unchanged."""
    torch.manual_seed(3)
    rank, H, nope, N, page = 40, 3, 24, 11, 64
    f, mag = freqs(ROT)
    pos = [0, 1, 63, 64, 65, 700, 5, 6, 7, 8, 9]
    seq = [0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1]
    table = i32([[3, 1, 7, 0, 2, 4, 5, 6, 8, 9, 10, 11], [12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23]])
    d = torch.randn(N, rank + rot_dim, device=DEV)
    norm_w = torch.randn(rank, device=DEV)
    pool = torch.zeros(24, 1, page, rank + rot_dim, device=DEV)
    st = status()
    ops.latent_kv_store(d, norm_w, f, mag, ROT["dims"], i32(seq), i32(pos), table, pool, page, rank, rot_dim, 1e-4, st)
    cos, sin = plain.rotary_tables(ROT, torch.tensor(pos), torch.float64)
    dd = d.double().cpu()
    c = plain.rms(dd[:, :rank], 1e-4) * norm_w.double().cpu()
    kr = plain.rotate(dd[:, rank:], cos, sin, ROT["dims"])
    for n in range(N):
        row = pool[int(table[seq[n], pos[n] // page]), 0, pos[n] % page].double().cpu()
        assert float((row[:rank] - c[n]).abs().max()) < 1e-5
        assert float((row[rank:] - kr[n]).abs().max()) < 2e-4 * (1 + pos[n] / 100)
        if rot_dim > ROT["dims"]:
            assert torch.equal(row[rank + ROT["dims"]:].float(), dd[n, rank + ROT["dims"]:].float())
    q = torch.randn(N, H * (nope + rot_dim), device=DEV)
    qx = torch.zeros(N, H * (rank + rot_dim), device=DEV)
    ops.latent_q_rotate(q, f, mag, ROT["dims"], i32(pos), qx, H, nope, rot_dim, rank)
    want = plain.rotate(q.double().cpu().view(N, H, nope + rot_dim)[..., nope:], cos, sin, ROT["dims"])
    got = qx.double().cpu().view(N, H, rank + rot_dim)
    assert float((got[..., rank:] - want).abs().max()) < 1e-3
    assert float(got[..., :rank].abs().max()) == 0.0
    assert int(st.item()) == 0


@pytest.mark.parametrize("a_dtype,w_dtype,o_dtype", [(torch.float32, torch.float32, torch.float32),
                                                     (torch.float32, torch.bfloat16, torch.bfloat16),
                                                     (torch.bfloat16, torch.bfloat16, torch.bfloat16)])
def test_per_head_product(a_dtype, w_dtype, o_dtype):
    torch.manual_seed(4)
    N, H, kin, nout, extra = 19, 5, 40, 24, 16
    a = torch.randn(N, H * (kin + extra), device=DEV).to(a_dtype)          # the heads' inputs are parts of wider heads
    w = torch.randn(H, nout, kin, device=DEV).to(w_dtype)
    out = torch.zeros(N, H * (nout + 3), device=DEV, dtype=o_dtype)
    ops.per_head_linear(a, H * (kin + extra), kin + extra, w, out, H * (nout + 3), nout + 3, N, H, kin, nout)
    want = torch.einsum("nhi,hji->nhj", a.double().view(N, H, kin + extra)[..., :kin], w.double())
    got = out.double().view(N, H, nout + 3)
    tol = 1e-5 if o_dtype == torch.float32 else 2 ** -7
    assert float((got[..., :nout] - want).abs().max()) <= tol * float(want.abs().max())
    assert float(got[..., nout:].abs().max()) == 0.0


def attention_reference(qx, rows, pos, window, scale, hdv):
    """qx [H, hdk], rows [pos + 1, hdk] (float64): the query at ``pos`` over its visible rows."""
    lo = max(0, pos - window + 1) if window else 0
    s = (qx @ rows[lo:pos + 1].T) * scale
    return torch.softmax(s, -1) @ rows[lo:pos + 1, :hdv]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,hdk,hdv,window", [(6, 64, 48, 37), (1, 24, 8, 1), (13, 168, 136, 0), (3, 576, 512, 200), (32, 96, 64, 136)])
def test_attention_over_cached_rows(dtype, H, hdk, hdv, window):
    torch.manual_seed(5 + H)
    page, L = 64, 300
    perm = torch.randperm(8)
    table = i32([perm.tolist()[:5] + [-1, -1, -1], perm.tolist()[5:] + [-1, -1, -1, -1, -1]])
    rows = torch.randn(2, L, hdk).to(dtype)
    pool = torch.zeros(8, 1, page, hdk, dtype=dtype, device=DEV)
    lens = [L, 130]
    for s in range(2):
        for j in range(lens[s]):
            pool[int(table[s, j // page]), 0, j % page] = rows[s, j].to(DEV)
    queries = [(0, 0), (0, 1), (0, 36), (0, 37), (0, 63), (0, 64), (0, 199), (0, 200), (0, 299), (1, 129), (1, 5)]
    N = len(queries)
    qx = (torch.randn(N, H * hdk) * 0.3).to(dtype)
    out = torch.zeros(N, H * hdv, dtype=dtype, device=DEV)
    st = status()
    scale = 0.21
    ops.attn_latent(qx.to(DEV), pool, out, i32([s for s, _ in queries]), i32([p for _, p in queries]), table, page, H, hdk, hdv,
                    window or None, scale, st)
    assert int(st.item()) == 0
    for n, (s, p) in enumerate(queries):
        want = attention_reference(qx[n].double().view(H, hdk), rows[s].double(), p, window, scale, hdv)
        tol = 2e-5 if dtype == torch.float32 else 2 ** -6
        assert float((out[n].double().cpu().view(H, hdv) - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (n, s, p)


@pytest.mark.parametrize("window", [0, 50, 136])
def test_attention_sees_exactly_its_window(window):
    """One key carries a score that dwarfs all others.  Placed on the last position inside the window (or, without
    a window, hundreds of positions back, behind several page borders) the output is that key's values; placed one
    position further back it must leave no trace."""
    H, hdk, hdv, page, pos = 2, 32, 16, 64, 400
    pool = torch.zeros(8, 1, page, hdk, device=DEV)
    table = i32([[7, 6, 5, 4, 3, 2, 1, 0]])
    base = torch.randn(pos + 1, hdk) * 0.1
    qx = torch.zeros(1, H * hdk, device=DEV)
    qx[0, 20] = 30.0
    qx[0, hdk + 20] = 30.0
    inside = pos - window + 1 if window else 3
    for place, seen in ((inside, True), (inside - 1, False)):
        if place < 0:
            continue
        rows = base.clone()
        rows[place, 20] = 30.0
        rows[place, :hdv] += 5.0
        for j in range(pos + 1):
            pool[int(table[0, j // page]), 0, j % page] = rows[j].to(DEV)
        out = torch.zeros(1, H * hdv, device=DEV)
        st = status()
        ops.attn_latent(qx, pool, out, i32([0]), i32([pos]), table, page, H, hdk, hdv, window or None, 1.0, st)
        got = out.cpu().view(H, hdv)
        if seen or not window:
            assert float((got - rows[place, :hdv]).abs().max()) < 1e-3
        else:
            assert float(got.abs().max()) < 1.0          # nothing of the key's values (about 5) came through


# ---------------------------------------------------------------------------------------------- the block's kernels
def test_scaled_add_norm_depth_average_and_activation():
    torch.manual_seed(6)
    N, D = 7, 100
    x = torch.randn(N, D, device=DEV)
    y = torch.randn(N, D, device=DEV)
    ys = torch.randn(D, device=DEV)
    gamma = torch.randn(D, device=DEV)
    h = torch.empty(N, D, device=DEV)
    x1 = x.clone()
    ops.add_rmsnorm(x1, y, gamma, h, 1e-5, yscale=ys)
    v = x.double() + y.double() * ys.double()
    assert float((x1.double() - v).abs().max()) < 1e-5
    assert float((h.double() - v / torch.sqrt((v ** 2).mean(-1, keepdim=True) + 1e-5) * gamma.double()).abs().max()) < 1e-4
    depth = 4
    hist = torch.randn(depth + 1, N, D, device=DEV)
    wts = torch.randn(depth + 1, device=DEV)
    for index, delta in ((2, y), (0, None)):
        hist2, x2 = hist.clone(), x.clone()
        ops.depth_mix(x2, delta, ys if delta is not None else None, hist2, wts, index)
        new = x.double() + (delta.double() * ys.double() if delta is not None else 0)
        assert float((hist2[index + 1].double() - new).abs().max()) < 1e-5
        want = sum(wts[j].double() * hist[j].double() for j in range(index + 1)) + wts[index + 1].double() * new
        assert float((x2.double() - want).abs().max()) < 1e-5
        assert torch.equal(hist2[index + 2:], hist[index + 2:]) and torch.equal(hist2[:index + 1], hist[:index + 1])
    z = torch.linspace(-6, 6, 1001, device=DEV)
    for p, q in ((0.3, -0.2), (-2.0, 1.5)):
        act = torch.empty_like(z)
        ops.xielu(z, torch.tensor([p, q], device=DEV), act)
        assert float((act.double().cpu() - plain.xielu(z.double().cpu(), p, q)).abs().max()) < 1e-5


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("H,hdk,hdv,window", [(6, 64, 48, 37), (1, 32, 16, 1), (13, 176, 144, 0), (3, 576, 512, 200),
                                              (32, 96, 64, 136), (40, 96, 64, 70), (16, 320, 256, 100)])
def test_attention_on_tensor_cores(H, hdk, hdv, window, splits):
    """The tensor-core form against float64: runs of new tokens behind cached ones, a run of five first tokens, single
    tokens, head counts that fill a tile, leave rows empty or need two tiles, with and without splitting the keys."""
    torch.manual_seed(7 + H)
    page = 64
    perm = torch.randperm(9).tolist()
    table = i32([perm[:5] + [-1, -1], perm[5:8] + [-1, -1, -1, -1], [perm[8]] + [-1] * 6])
    lens, pasts = [290, 131, 5], [100, 130, 0]
    rows = torch.randn(3, 300, hdk).to(torch.bfloat16)
    pool = torch.zeros(9, 1, page, hdk, dtype=torch.bfloat16, device=DEV)
    for s in range(3):
        for j in range(lens[s]):
            pool[int(table[s, j // page]), 0, j % page] = rows[s, j].to(DEV)
    news = [lens[s] - pasts[s] for s in range(3)]
    N = sum(news)
    starts = np.concatenate([[0], np.cumsum(news)])
    qx = (torch.randn(N, H * hdk) * 0.3).to(torch.bfloat16)
    hg = ops.attn_latent_mma_heads(H)
    tq = 32 // hg
    tiles = [(s, f) for s in range(3) for f in range(0, news[s], tq)]
    out = torch.zeros(N, H * hdv, dtype=torch.bfloat16, device=DEV)
    st = status()
    part_o = torch.empty(N, H, splits, hdv, device=DEV) if splits > 1 else None
    part_ml = torch.empty(N, H, splits, 2, device=DEV) if splits > 1 else None
    ops.attn_latent_mma(qx.to(DEV), pool, out, i32([t[0] for t in tiles]), i32([t[1] for t in tiles]), i32(starts), i32(pasts),
                        table, page, H, hdk, hdv, window or None, 0.21, st, splits, 2, part_o, part_ml)
    assert int(st.item()) == 0
    worst = 0.0
    for s in range(3):
        for t in range(news[s]):
            n = starts[s] + t
            want = attention_reference(qx[n].double().view(H, hdk), rows[s].double(), pasts[s] + t, window, 0.21, hdv)
            err = float((out[n].double().cpu().view(H, hdv) - want).abs().max()) / max(1.0, float(want.abs().max()))
            worst = max(worst, err)
            assert err <= 2 ** -6, (s, t, err)


@pytest.mark.parametrize("mode", [ops.SCAN_DECAY_BONUS, ops.SCAN_LOWER_SIGMOID])
def test_gates_made_ahead_give_the_same_bits(mode):
    torch.manual_seed(8)
    H, K, V, T = 3, 48, 40, 70
    q, k, g = (torch.randn(T, H * K, device=DEV) for _ in range(3))
    v = torch.randn(T, H * V, device=DEV)
    bias, lower, bonus = torch.randn(H * K, device=DEV), torch.rand(H * K, device=DEV), torch.randn(H * K, device=DEV)
    outs, states = [], []
    for ahead in (False, True):
        state = torch.zeros(2, H * K * V, device=DEV)
        out = torch.zeros(T, H * V, device=DEV)
        if ahead:
            made = torch.zeros(3, T, H * K, device=DEV)
            if mode == ops.SCAN_DECAY_BONUS:
                ops.gate_prepare(mode, None, g, bias, None, None, None, made[2])
                ops.gated_scan(mode, q, k, made[2], v, None, None, bonus, state, i32([0, T]), i32([1]), out, 1, H, K, V, ready=True)
            else:
                ops.gate_prepare(mode, q, g, bias, lower, made[0], made[1], made[2])
                ops.gated_scan(mode, made[0], made[1], made[2], v, None, None, None, state, i32([0, T]), i32([1]), out, 1, H, K, V,
                               ready=True)
        else:
            ops.gated_scan(mode, q, k if mode == ops.SCAN_DECAY_BONUS else None, g, v, bias, lower if mode else None,
                           bonus if not mode else None, state, i32([0, T]), i32([1]), out, 1, H, K, V)
        outs.append(out)
        states.append(state)
    assert torch.equal(outs[0], outs[1]) and torch.equal(states[0], states[1])


def test_activation_in_the_products_epilogue():
    """The weight-streaming product with xIELU in its epilogue against the product followed by the activation's kernel."""
    torch.manual_seed(9)
    rows, K, N = 5, 96, 200
    a = torch.randn(rows, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    pq = torch.tensor([0.4, -0.3], device=DEV)
    fused = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm_skinny(a, w, fused, xielu_pq=pq)
    z = torch.empty(rows, N, device=DEV)
    ops.gemm_skinny(a, w, z)
    two = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)
    ops.xielu(z, pq, two)
    want = plain.xielu(a.double().cpu() @ w.double().cpu().T, 0.4, -0.3)
    assert float((fused.double().cpu() - want).abs().max()) <= 2 ** -7 * float(want.abs().max())
    assert float((fused.float() - two.float()).abs().max()) <= 2 ** -7 * float(want.abs().max())
