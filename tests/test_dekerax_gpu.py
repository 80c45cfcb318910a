"""The Dekerax decoder on the GPU against the plain implementation: every new kernel alone against a float64 loop
written here from its formula, then whole models (tiny configurations that differ in every size) replayed whole, with
the last tokens one by one, in portions down to two tokens, and mixed in a pool so small that pages and state slots are
used again; window edges in prompts and in decoding; decoding from CUDA graphs; greedy generation through
`Engine.generate` and the scheduler.  In 32-bit every schedule must give the same bits: a difference under one schedule
only is a fault of the cache, the state or the batch."""

import copy

import pytest
import torch

from tests.gpu_helpers import BF16, F32, assert_close, i32, table_tensor
from tests.plain import dekerax_plain as plain_model
from tests.plain.dekerax_plain import PlainDekerax, forward, greedy_generate
from tests.test_replay_gpu import cuts_changing, cuts_last32, cuts_whole, replay, steps_alone, steps_decode_together, steps_mixed
from tests.tiny import random_tokens
from tests.tiny_dekerax import CONFIGS, PAGE_SIZE, write_tiny_dekerax

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]
F32_ATOL = 5e-5
BF16_REL = 0.05
LENGTHS = {"D1": [1, 5, 17, 70, 33, 130, 64], "D2": [7, 40, 64, 97, 2, 150]}
F64 = torch.float64


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def unit(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("H", [48, 203, 1024])
def test_normalised_addend_residual_sum_and_norm(adt, H):
    """x += a / rms(a) * w1 (+ a row); h = x / rms(x) * w2; with picked rows x stays; without an addend; the sum only."""
    from tensorline_b200 import ops
    T, eps = 9, 1e-5
    x0, a = rnd(T, H, seed=1, scale=3.0), rnd(T, H, seed=2, scale=0.1, dtype=adt)
    w1, w2 = (1 + rnd(H, seed=3, scale=0.2)).to(torch.bfloat16), (1 + rnd(H, seed=4, scale=0.2)).to(torch.bfloat16)
    row = rnd(H, seed=5, scale=2.0)
    tol = F32 if adt == torch.float32 else BF16
    for extra in (None, row):
        want_x = x0.double() + unit(a.double(), eps) * w1.double() + (0 if extra is None else extra.double())
        want_h = unit(want_x, eps) * w2.double()
        x, h = x0.clone().cuda(), torch.empty(T, H, dtype=adt, device="cuda")
        ops.post_norm_add_norm(x, a.cuda(), w1.cuda(), w2.cuda(), h, eps, extra=None if extra is None else extra.cuda())
        assert_close(x, want_x, "stream", **F32)
        assert_close(h, want_h, "norm", **tol)
        rows = i32([7, 0, 3])
        x2, h2 = x0.clone().cuda(), torch.empty(3, H, dtype=adt, device="cuda")
        ops.post_norm_add_norm(x2, a.cuda(), w1.cuda(), w2.cuda(), h2, eps, extra=None if extra is None else extra.cuda(), rows=rows)
        assert torch.equal(x2.cpu(), x0) and torch.equal(h2, h[rows.long()])
    x, h = x0.clone().cuda(), torch.empty(T, H, dtype=adt, device="cuda")
    ops.post_norm_add_norm(x, None, None, w2.cuda(), h, eps, extra=row.cuda())
    assert_close(x, x0.double() + row.double(), "row only", **F32)
    assert_close(h, unit(x0.double() + row.double(), eps) * w2.double(), "norm after a row", **tol)
    x = x0.clone().cuda()
    ops.post_norm_add_norm(x, a.cuda(), w1.cuda(), None, None, eps)
    assert_close(x, x0.double() + unit(a.double(), eps) * w1.double(), "sum only", **F32)


@pytest.mark.parametrize("adt", DT)
def test_gelu_gate(adt):
    from tensorline_b200 import ops
    gu = rnd(37, 2 * 72, seed=1, scale=2.0, dtype=adt)
    out = torch.empty(37, 72, dtype=adt, device="cuda")
    ops.silu_mul(gu.cuda(), out, act="gelu_tanh")
    want = plain_model.gelu_tanh(gu[:, :72].double()) * gu[:, 72:].double()
    assert_close(out, want, "gelu_tanh(gate) * up", **(F32 if adt == torch.float32 else BF16))


@pytest.mark.parametrize("T", [8, 37, 700])
def test_gelu_gate_in_the_epilogue_of_the_tensor_core_products(T):
    """Both tcgen05 products with the tanh form of gelu in their epilogue: bit for bit the product, stored in bfloat16,
    followed by the activation kernel, and the formula in float64."""
    from tensorline_b200 import ops, ops_gemm
    I, K = 320, 520
    x = rnd(T, K, seed=1, dtype=torch.bfloat16).cuda()
    g, u = rnd(I, K, seed=2, scale=0.1, dtype=torch.bfloat16), rnd(I, K, seed=3, scale=0.1, dtype=torch.bfloat16)
    w = torch.stack((g.view(I // 64, 64, K), u.view(I // 64, 64, K)), dim=1).reshape(2 * I, K).contiguous().cuda()
    if T <= 64:
        kw = dict(swap=1, bn=16 if T <= 16 else 64, splits=1)
        got, gu = ops_gemm.gemm_tc(x, w, gated="gelu_tanh", **kw), ops_gemm.gemm_tc(x, w, **kw)
    else:
        got, gu = ops_gemm.gemm_tc2(x, w, gated="gelu_tanh"), ops_gemm.gemm_tc2(x, w)
    ops_gemm.check_status()
    two_pass = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    ops.silu_mul(gu, two_pass, block=64, act="gelu_tanh")
    assert torch.equal(got, two_pass)
    gd, ud = x.double().cpu() @ g.double().T, x.double().cpu() @ u.double().T
    assert_close(got, plain_model.gelu_tanh(gd) * ud, "gelu_tanh(gate) * up", rtol=3e-2, atol=3e-2)
    with pytest.raises(ops.KernelError, match="gelu"):
        ops_gemm.gemm_tc2(x, w, gated="gelu")


def _conv_plain(x, w, lens):
    """x [T, C] rows in request order; per request a causal convolution over time, then silu."""
    out, t0 = torch.zeros_like(x), 0
    for n in lens:
        out[t0:t0 + n] = plain_model.short_convolution(x[t0:t0 + n], w)
        t0 += n
    return torch.nn.functional.silu(out)


def _run_in_cuts(lens, cuts, slots, step):
    """Calls step(rows, q_start, live slots) for every launch of a schedule: cut[b] tokens of request b (0: left out)."""
    B = len(lens)
    starts = [sum(lens[:b]) for b in range(B)]
    done = [0] * B
    for cut in cuts:
        rows, q_start, live = [], [0], []
        for b in range(B):
            n = min(cut[b], lens[b] - done[b])
            if n > 0:
                rows += list(range(starts[b] + done[b], starts[b] + done[b] + n)); done[b] += n
                q_start.append(len(rows)); live.append(slots[b])
        if rows:
            step(rows, q_start, live)
    assert done == list(lens)


CUTS = [[1000] * 4, [1, 5, 2, 3], [2, 2, 2, 2], [16, 1, 0, 7], [3, 16, 16, 16], [1, 1, 1, 1], [40, 40, 40, 40], [1000] * 4]
CUTS_SINGLE = [[1, 1, 1, 1]] * 140


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("nqk,d,nv,dv,taps", [(2, 8, 4, 24, 4), (1, 40, 1, 72, 2), (2, 136, 2, 8, 1), (2, 20, 6, 12, 3), (5, 8, 5, 8, 5)])
def test_convolution_silu_unit_length_in_one_step_and_in_portions(adt, nqk, d, nv, dv, taps):
    """Whole requests against the formula; the same requests in portions (down to single tokens, shorter than the taps) with
    the last inputs left in the slots: the same bits."""
    from tensorline_b200 import ops
    lens = [37, 1, 5, 70]
    T, C = sum(lens), 2 * nqk * d + nv * dv
    proj = rnd(T, C + 7, seed=1, dtype=adt)                     # columns that belong to nobody behind q | k | v
    w = rnd(C, taps, seed=2, scale=0.7, dtype=torch.bfloat16)
    y = _conv_plain(proj[:, :C].double(), w.double(), lens)
    q, k = y[:, :nqk * d].view(T, nqk, d), y[:, nqk * d:2 * nqk * d].view(T, nqk, d)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    want = torch.cat([q.reshape(T, -1), k.reshape(T, -1), y[:, 2 * nqk * d:]], dim=1)
    slots = [5, 0, 3, 2]

    def run(cuts):
        state = torch.zeros(7, max(1, (taps - 1) * C), device="cuda")
        state[1] = 7.0                                          # a slot nobody owns: must stay as it is
        out = torch.zeros(T, C, device="cuda")

        def step(rows, q_start, live):
            idx = torch.tensor(rows)
            part = torch.zeros(len(rows), C, device="cuda")
            longest = max(b - a for a, b in zip(q_start, q_start[1:]))
            ops.conv_prep(proj[idx].contiguous().cuda(), w.cuda(), state if taps > 1 else None, i32(q_start), i32(live), part,
                          B=len(live), max_q_len=longest, nqk=nqk, d=d, nv=nv, dv=dv, unit_eps=1e-6, q_scale=d ** -0.5)
            out[idx.cuda()] = part
        _run_in_cuts(lens, cuts, slots, step)
        assert bool((state[1] == 7.0).all()) and bool((state[[4, 6]] == 0).all())
        return out

    whole = run(CUTS[:1])
    assert_close(whole, want, "convolution, silu, unit length", rtol=2e-5, atol=2e-5)
    assert torch.equal(run(CUTS[1:]), whole)


def _delta_plain(q, k, v, beta, g, lens):
    """q, k [T, nqk, d], v [T, H, dv], beta, g [T, H]; per request and head the recurrence of the module text."""
    T, H, dv = v.shape
    nqk, d = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, dv, dtype=F64)
    t0 = 0
    for n in lens:
        S = torch.zeros(H, d, dv, dtype=F64)
        for t in range(t0, t0 + n):
            for h in range(H):
                j = h // (H // nqk)
                S[h] = g[t, h] * S[h]
                u = beta[t, h] * (v[t, h] - S[h].T @ k[t, j])
                S[h] = S[h] + torch.outer(k[t, j], u)
                out[t, h] = S[h].T @ q[t, j]
        t0 += n
    return out


def _gates_plain(gates, A_log, dt_bias, H):
    beta = torch.sigmoid(gates[:, :H].double())
    g = torch.exp(-torch.exp(A_log.double()) * torch.nn.functional.softplus(gates[:, H:2 * H].double() + dt_bias.double()))
    return beta, g


@pytest.mark.parametrize("pair", [False, True], ids=["float", "pair"])
@pytest.mark.parametrize("H,nqk,d,dv", [(4, 2, 8, 24), (1, 1, 40, 72), (2, 2, 136, 8), (6, 2, 20, 12), (3, 1, 256, 16), (2, 2, 64, 33)])
def test_delta_rule_in_one_step_and_in_portions(H, nqk, d, dv, pair):
    """The recurrence over whole requests in one launch against the formula, and the same requests cut into portions
    (single tokens among them) over several launches with the state left in the slots: the same bits.  `pair`: the state as
    the 32-bit engine keeps it, two floats an element."""
    from tensorline_b200 import ops
    lens = [37, 1, 5, 70]
    T, C = sum(lens), 2 * nqk * d + H * dv
    qkv = rnd(T, C, seed=1)
    qk = qkv[:, :2 * nqk * d].view(T, 2 * nqk, d)
    qkv[:, :2 * nqk * d] = (qk / qk.norm(dim=-1, keepdim=True)).reshape(T, -1)
    gates = rnd(T, 2 * H + 3, seed=2, scale=2.0)
    A_log, dt_bias = torch.linspace(-5.0, -1.0, H), torch.linspace(-1.0, 1.0, H)
    beta, g = _gates_plain(gates, A_log, dt_bias, H)
    want = _delta_plain(qkv[:, :nqk * d].double().view(T, nqk, d), qkv[:, nqk * d:2 * nqk * d].double().view(T, nqk, d),
                        qkv[:, 2 * nqk * d:].double().view(T, H, dv), beta, g, lens).reshape(T, H * dv)
    per_slot = H * -(-dv // ops.delta_columns()) * ops.delta_state_floats(d, pair)
    assert ops.delta_state_floats(d, True) == 2 * ops.delta_state_floats(d, False)
    slots = [5, 0, 3, 2]

    def run(cuts):
        state = torch.zeros(7, per_slot, device="cuda")
        state[1] = 7.0
        out = torch.zeros(T, H * dv, device="cuda")

        def step(rows, q_start, live):
            idx = torch.tensor(rows)
            part = torch.zeros(len(rows), H * dv, device="cuda")
            ops.delta_scan(qkv[idx].contiguous().cuda(), gates[idx].contiguous().cuda(), A_log.cuda(), dt_bias.cuda(), state,
                           i32(q_start), i32(live), part, B=len(live), H=H, nqk=nqk, d=d, dv=dv, compensated=pair)
            out[idx.cuda()] = part
        _run_in_cuts(lens, cuts, slots, step)
        assert bool((state[1] == 7.0).all()) and bool((state[[4, 6]] == 0).all())
        return out

    whole = run(CUTS[:1])
    assert_close(whole, want, "delta rule", rtol=5e-5, atol=5e-5)
    assert torch.equal(run(CUTS[1:]), whole)
    assert torch.equal(run(CUTS_SINGLE), whole)


def test_a_pair_of_floats_keeps_the_state_exact_over_many_tokens():
    """1,500 tokens, most of them one of three that come again and again, with decays just under one.  A decay rounded to a float
    is off by the same 3e-8 whenever its token comes again, so the weight of a far token, a product of a thousand decays, drifts
    from the float64 recurrence by 1e-5 and more, and a float state gathers a rounding a token on top; with pairs of floats for
    the state and the decay (the 32-bit engine) the read-out stays at the accuracy of the sums that feed it."""
    from tensorline_b200 import ops
    H, nqk, d, dv, T = 2, 1, 32, 48, 1500
    kinds = rnd(3, 2 * nqk * d + H * dv, seed=7)
    which = torch.randint(0, 3, (T,), generator=torch.Generator().manual_seed(9))
    qkv = kinds[which].clone()
    qkv[::50] = rnd(T // 50, qkv.shape[1], seed=10)              # now and then another token
    qk = qkv[:, :2 * nqk * d].view(T, 2 * nqk, d)
    qkv[:, :2 * nqk * d] = (qk / qk.norm(dim=-1, keepdim=True)).reshape(T, -1)
    gates = rnd(3, 2 * H, seed=8)[which].contiguous()
    A_log, dt_bias = torch.tensor([-7.0, -6.0]), torch.zeros(H)
    beta, g = _gates_plain(gates, A_log, dt_bias, H)
    want = _delta_plain(qkv[:, :d].double().view(T, 1, d), qkv[:, d:2 * d].double().view(T, 1, d), qkv[:, 2 * d:].double().view(T, H, dv),
                        beta, g, [T])
    errs = {}
    for pair in (False, True):
        state = torch.zeros(2, H * -(-dv // ops.delta_columns()) * ops.delta_state_floats(d, pair), device="cuda")
        out = torch.zeros(T, H * dv, device="cuda")
        ops.delta_scan(qkv.cuda(), gates.cuda(), A_log.cuda(), dt_bias.cuda(), state, i32([0, T]), i32([1]), out, B=1, H=H, nqk=nqk,
                       d=d, dv=dv, compensated=pair)
        e = (out.double().cpu().view(T, H, dv) - want)[-200:]
        errs[pair] = float(e.pow(2).sum().sqrt() / want[-200:].pow(2).sum().sqrt())
    assert errs[True] < 3e-6 and errs[True] < 0.25 * errs[False], errs


@pytest.mark.parametrize("decoded", [0, 300])
def test_delta_rule_keeps_a_far_token(decoded):
    """One token writes a value under a key nobody else uses; 700 tokens later (the last `decoded` of them one launch
    each) a query along that key reads it back, decayed by the product of the gates in between and by nothing else."""
    from tensorline_b200 import ops
    H, nqk, d, dv, T, mark = 2, 1, 32, 24, 702, 1
    g0 = torch.Generator().manual_seed(3)
    k = torch.randn(T, d, generator=g0)
    k[:, 0] = 0.0
    k = k / k.norm(dim=-1, keepdim=True)
    k[mark] = 0.0; k[mark, 0] = 1.0
    q = k.clone()
    q[-1] = 0.0; q[-1, 0] = 1.0
    v = torch.randn(T, H * dv, generator=g0)
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    gates = torch.randn(T, 2 * H, generator=g0)
    gates[mark, :H] = 30.0                                     # beta = 1: the value is written whole
    A_log, dt_bias = torch.tensor([-7.0, -5.0]), torch.zeros(H)
    _, g = _gates_plain(gates, A_log, dt_bias, H)
    want = v[mark].double().view(H, dv) * g[mark + 1:].prod(0)[:, None]
    assert float(want.abs().max()) > 0.5                      # the far token is what the last query reads, and it is not small
    state = torch.zeros(2, H * -(-dv // ops.delta_columns()) * ops.delta_state_floats(d), device="cuda")
    out = torch.zeros(T, H * dv, device="cuda")
    cuts = [T - decoded] + [1] * decoded
    t0 = 0
    for n in cuts:
        ops.delta_scan(qkv[t0:t0 + n].contiguous().cuda(), gates[t0:t0 + n].contiguous().cuda(), A_log.cuda(), dt_bias.cuda(), state,
                       i32([0, n]), i32([1]), out[t0:t0 + n], B=1, H=H, nqk=nqk, d=d, dv=dv)
        t0 += n
    assert_close(out[-1].view(H, dv), want, "the far token's value", rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("H,K,N,xs,ys", [(3, 16, 24, 24, 40), (2, 40, 24, 40, 24), (1, 7, 130, 9, 131), (8, 128, 64, 160, 64)])
def test_product_per_head(adt, H, K, N, xs, ys):
    from tensorline_b200 import ops
    T = 21
    x, w = rnd(T, H * xs, seed=1, dtype=adt), rnd(H, K, N, seed=2, scale=0.3, dtype=torch.bfloat16)
    y = torch.full((T, H * ys), 5.0, dtype=adt, device="cuda")
    ops.head_matmul(x.cuda(), w.cuda(), y, H, K, N, xs, ys)
    want = torch.einsum("thk,hkn->thn", x.double().view(T, H, xs)[:, :, :K], w.double())
    assert_close(y.view(T, H, ys)[:, :, :N], want, "per-head product", **(F32 if adt == torch.float32 else BF16))
    assert bool((y.view(T, H, ys)[:, :, N:] == 5.0).all())     # what lies between the heads is nobody's
    one = torch.zeros(1, H * ys, dtype=adt, device="cuda")     # a row's result does not depend on the other rows
    ops.head_matmul(x[13:14].cuda(), w.cuda(), one, H, K, N, xs, ys)
    assert torch.equal(one.view(H, ys)[:, :N], y.view(T, H, ys)[13, :, :N])


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("qr,rank,dr,rot,d,page", [(20, 24, 8, 8, 32, 8), (36, 40, 16, 8, 64, 16), (8, 12, 4, 4, 16, 4), (5, 7, 6, 0, 13, 2)])
def test_latent_rows_into_pages_and_rotated_queries(adt, qr, rank, dr, rot, d, page):
    """Both norms, the rotation of the shared key part at every token's own position, the page write through a scattered
    table; then the query rows' rotated part."""
    from tensorline_b200 import ops
    if adt == torch.bfloat16 and d % 8:
        pytest.skip("bfloat16 pages are padded to multiples of 16")
    T, eps, base = 23, 1e-5, 100.0
    down = rnd(T, qr + rank + dr, seed=1)
    wq, wkv = (1 + rnd(qr, seed=2, scale=0.2)).to(torch.bfloat16), (1 + rnd(rank, seed=3, scale=0.2)).to(torch.bfloat16)
    pos = [40 + t for t in range(15)] + [3 + t for t in range(8)]               # two requests, the first resumed at 40
    slot = [2] * 15 + [0] * 8
    inv_freq = (base ** (-torch.arange(0, rot, 2, dtype=F64) / rot)).float() if rot else torch.zeros(0)
    n_pages = 40
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).tolist()
    rows = [order[:-(-16 // page)], [], order[8:8 + -(-55 // page)]]
    table = table_tensor(rows, -(-64 // page), n_pages)
    pages = torch.full((n_pages + 1, 1, page, d), 9.0, dtype=adt, device="cuda")
    cq = torch.empty(T, qr, dtype=adt, device="cuda")
    ops.latent_prep(down.cuda(), qr, rank, dr, wq.cuda(), wkv.cuda(), eps, inv_freq.cuda(), rot, i32(pos), i32(slot), table, page, cq, pages)
    tol = F32 if adt == torch.float32 else BF16
    assert_close(cq, unit(down[:, :qr].double(), eps) * wq.double(), "query latent", **tol)
    lat = unit(down[:, qr:qr + rank].double(), eps) * wkv.double()
    shared = plain_model.turn(down[:, None, qr + rank:].double(), pos, rot, base)[:, 0]
    want = torch.cat([lat, shared, torch.zeros(T, d - rank - dr, dtype=F64)], dim=1)
    seen = set()
    for t in range(T):
        pg = rows[slot[t]][pos[t] // page]
        assert_close(pages[pg, 0, pos[t] % page], want[t], f"page row of token {t}", **tol)
        seen.add((pg, pos[t] % page))
    untouched = [(p, o) for p in range(n_pages + 1) for o in range(page) if (p, o) not in seen]
    assert all(bool((pages[p, 0, o] == 9.0).all()) for p, o in untouched[::7])
    H, dk = 3, 10
    q = rnd(T, H * (dk + dr), seed=6, dtype=adt)
    qa = torch.full((T, H * d), 4.0, dtype=adt, device="cuda")
    ops.latent_qrot(q.cuda(), dk, dr, inv_freq.cuda(), rot, i32(pos), qa, rank, H)
    turned = plain_model.turn(q.double().view(T, H, dk + dr)[:, :, dk:], pos, rot, base)
    assert_close(qa.view(T, H, d)[:, :, rank:rank + dr], turned, "rotated query part", **tol)
    assert bool((qa.view(T, H, d)[:, :, :rank] == 4.0).all()) and bool((qa.view(T, H, d)[:, :, rank + dr:] == 0).all())


@pytest.mark.parametrize("E,top", [(5, 2), (3, 1), (64, 8), (9, 9)])
def test_choice_of_experts_by_sigmoid_scores(E, top):
    from tensorline_b200 import ops
    T = 33
    z = rnd(T, E + 1, seed=E, scale=2.0).cuda()               # one more column behind the experts' (a shared expert's gate)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    ops.topk_softmax(z[:, :E], top, idx, wts, scoring="sigmoid")
    val, want_idx = torch.topk(z[:, :E].double().cpu(), top, dim=1)
    assert torch.equal(idx.cpu().long(), want_idx)
    assert_close(wts, torch.sigmoid(val), "scores of the chosen experts, not renormalised", **F32)


def _gated_experts_plain(h, gate_up, down, idx, wts, shared, sg):
    T, top = idx.shape
    F = down.shape[2]
    silu = torch.nn.functional.silu
    out = torch.zeros(T, down.shape[1], dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            x = wts[t, j] * h[t]                                 # the weight is on the expert's input
            out[t] += down[e] @ (silu(gate_up[e, :F] @ x) * (gate_up[e, F:] @ x))
    return out + torch.sigmoid(sg)[:, None] * shared


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("T,K,F,E,top", [(5, 48, 40, 5, 2), (70, 72, 16, 9, 4), (3, 52, 21, 3, 1), (200, 64, 24, 6, 3)])
def test_gated_experts_weighted_on_their_input_streamed_and_sorted(adt, T, K, F, E, top):
    """Both routes of the experts' products with the options this design sets: gate and up rows stacked, silu, the weight on
    the input, an unweighted sum, and a gated addend a token."""
    from tensorline_b200 import ops
    h = rnd(T, K, seed=1, dtype=adt)
    gu, dn = rnd(E, 2 * F, K, seed=2, scale=0.2, dtype=torch.bfloat16), rnd(E, K, F, seed=3, scale=0.2, dtype=torch.bfloat16)
    z = rnd(T, E + 1, seed=4, scale=2.0)
    shared = rnd(T, K, seed=5, dtype=adt)
    val, idx = torch.topk(z[:, :E], top, dim=1)
    wts = torch.sigmoid(val).contiguous()
    want = _gated_experts_plain(h.double(), gu.double(), dn.double(), idx, wts.double(), shared.double(), z[:, E].double())
    hd, gud, dnd, idd, wd, zd, sd = h.cuda(), gu.cuda(), dn.cuda(), idx.to(torch.int32).cuda(), wts.cuda(), z.cuda(), shared.cuda()
    tol = F32 if adt == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    a = torch.empty(T * top, F, dtype=adt, device="cuda")
    y = torch.empty(T, K, dtype=adt, device="cuda")
    ops.moe_up(hd, gud, idd, a, act="silu", gated=True, in_scale=wd)
    ops.moe_down(a, dnd, idd, None, y, extra=sd, extra_gate=zd[:, E])
    assert_close(y, want, "streamed", **tol)
    offsets, place_of, pair_at = ops.moe_sort(idd, E)
    bounds = offsets.tolist()
    cap = -(-max(b - a_ for a_, b in zip(bounds, bounds[1:])) // 8) * 8
    rows = torch.empty(E * cap, K, dtype=adt, device="cuda")
    ops.moe_gather(hd, pair_at, idd, offsets, top, rows, cap=cap, scale=wd.view(-1))
    inner = torch.bmm(rows.view(E, cap, K).float(), gud.float().transpose(1, 2)).to(adt)
    act = torch.empty(E * cap, F, dtype=adt, device="cuda")
    ops.silu_mul(inner.view(E * cap, 2 * F), act, act="silu")
    outs = torch.bmm(act.view(E, cap, F).float(), dnd.float().transpose(1, 2)).to(adt)
    y2 = torch.empty(T, K, dtype=adt, device="cuda")
    ops.moe_combine(outs.view(E * cap, K), place_of, idd, offsets, None, y2, cap=cap, extra=sd, extra_gate=zd[:, E])
    assert_close(y2, want, "sorted", **tol)


# ------------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module", params=["D1", "D2"])
def model(request, tmp_path_factory):
    name = request.param
    folder = write_tiny_dekerax(name, tmp_path_factory.mktemp(f"tiny_{name}"))
    plain = PlainDekerax(folder)
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": random_tokens(V, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    want = {rid: forward(plain, toks) for rid, toks in reqs.items()}
    return dict(name=name, folder=folder, reqs=reqs, want=want, page=PAGE_SIZE[name], vocab=V, plain=plain)


def check(model, dtype, got, what):
    """32-bit: every position within F32_ATOL (times the largest |logit| where that is above one).  bfloat16: the largest logit
    error of a position as a share of the request's largest |logit|: four positions in five within BF16_REL, every one within
    that largest |logit|.  (Measured on a 130-token request: median 0.014 / 0.006, nine in ten under 0.044 / 0.009, largest
    0.27 / 0.016 for D1 / D2; the residual stream drifts by 0.003 to 0.005 a layer and jumps where a sigmoid score near a tie
    picks another expert, with the same mixers before and after the jump.  The 32-bit runs pin those positions.)"""
    assert got, "nothing was compared"
    over = 0
    for (rid, p), row in got.items():
        ref = model["want"][rid][p]
        err = float((row - ref).abs().max())
        if dtype == "float32":
            bound = F32_ATOL * max(1.0, float(ref.abs().max()))
            assert err <= bound, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {bound:.3e}"
        else:
            top = float(model["want"][rid].abs().max())
            assert err <= top, f"{what}: request {rid} position {p}: max abs err {err:.3e} > {top:.3e}"
            over += err > BF16_REL * top
    assert over <= 0.2 * len(got), f"{what}: {over} of {len(got)} positions are beyond the bfloat16 bound"


def test_the_model_is_chosen_by_its_configuration_and_every_layer_matches(model):
    """Residual stream after every layer that runs (a looped layer counts each time), 32-bit engine against the plain model."""
    from tensorline_b200.replay import TraceSession, make_runner
    runner, cfg = make_runner(model["folder"], "float32", 256, page_size=model["page"], max_live=2)
    assert type(cfg).__name__ == "DekeraxConfig" and cfg.to_json_dict() == CONFIGS[model["name"]]
    seen = []
    for blk in runner.model.blocks:
        def fwd(x, pending, ctx, cache, orig=blk.forward):
            out = orig(x, pending, ctx, cache)
            after = x.clone()
            out.add_into(after)
            seen.append(after.double().cpu())
            return out
        blk.forward = fwd
    toks = model["reqs"]["r2"]
    TraceSession(runner).run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    want = []
    forward(model["plain"], toks, want)
    assert len(seen) == len(want) == len(cfg.run_order()) > len(CONFIGS[model["name"]]["layers"])
    for i, (g, w) in enumerate(zip(seen, want)):
        assert_close(g, w, f"residual stream after layer run {i}", rtol=5e-5, atol=5e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_schedules_agree_with_the_plain_model(model, dtype):
    results = {}
    for what, cuts in (("whole", cuts_whole), ("last 32 one by one", cuts_last32), ("changing portions", cuts_changing)):
        results[what] = replay(model, dtype, steps_alone(model, cuts), max_tokens=192)
        check(model, dtype, results[what], what)
        assert len(results[what]) == sum(len(t) for t in model["reqs"].values())
    for seed in (1, 2):
        steps, peak = steps_mixed(model, seed)
        assert max(len(s["entries"]) for s in steps) >= 3
        total = sum(-(-len(t) // model["page"]) * model["page"] for t in model["reqs"].values())
        assert peak < total, "the pool must be too small to hold all requests: pages and slots have to be used again"
        results[f"mixed {seed}"] = replay(model, dtype, steps, max_tokens=peak)
        check(model, dtype, results[f"mixed {seed}"], f"mixed {seed}")
        assert len(results[f"mixed {seed}"]) == len(results["whole"])
    if dtype == "float32":                                  # one order of additions per position
        for what, got in results.items():
            for key, row in got.items():
                assert torch.equal(row, results["whole"][key]), f"{what} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(model, dtype):
    """A one-token prompt, then 150 tokens decoded one by one: states and windows are carried through 150 launches, and
    every window passes over decoded tokens and over page borders."""
    toks = random_tokens(model["vocab"], 151, seed=7)
    want = forward(model["plain"], toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = ["x"]
    m2 = dict(model, reqs={"x": toks}, want={"x": want})
    got = replay(m2, dtype, steps, max_tokens=160)
    check(m2, dtype, got, "token by token")
    assert sorted(p for _, p in got) == list(range(151))


def _other_windows(raw, by):
    """The configuration with every window `by` tokens wider."""
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if "mask" in layer["mixer"]:
            layer["mixer"]["mask"]["size"] += by
    return raw


def test_window_edges_in_prompts_and_in_decoding(model, tmp_path):
    """The plain model with every window one token wider or narrower gives other logits from the first position a window
    cuts on (so a key that is wrongly seen, or wrongly not seen, shows), and the engine follows the right one: whole, with the
    tokens around every window's edge decoded one by one, and in portions that end on both sides of the edges."""
    toks = random_tokens(model["vocab"], 90, seed=11)
    right = forward(model["plain"], toks)
    windows = sorted({l["mixer"]["mask"]["size"] for l in CONFIGS[model["name"]]["layers"] if "mask" in l["mixer"]})
    first = windows[0]                                      # the first position whose smallest window leaves a key out
    for by in (-1, 1):
        other = PlainDekerax(model["folder"])
        other.cfg = _other_windows(other.cfg, by)
        wrong = forward(other, toks)
        gap = (wrong - right).abs().max(1).values
        assert float(gap[:first - 1].max()) == 0.0
        assert float(gap[first]) > 100 * F32_ATOL and float(gap[first:].median()) > 100 * F32_ATOL, \
            "the plain model must tell a window that is one token off"
    m2 = dict(model, reqs={"w": toks}, want={"w": right})
    edges = sorted({w + k for w in windows for k in (-1, 0, 1)})
    cuts = [[90], [windows[0] - 1] + [1] * (91 - windows[0]), [e2 - e1 for e1, e2 in zip([0] + edges, edges + [90]) if e2 > e1]]
    for dtype in ("float32", "bfloat16"):
        for c in cuts:
            assert sum(c) == 90
            got = replay(m2, dtype, steps_alone(m2, lambda n, c=c: c), max_tokens=96)
            check(m2, dtype, got, f"window edges, portions {c[:4]}...")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_agree_with_eager_steps(model, dtype):
    """Steps of single tokens replayed from CUDA graphs (state slots are fixed addresses, padding rows use the spare
    slot): three live requests in the bucket of four, shrinking as they end; 32-bit: the bits of the eager steps."""
    rids = ["r3", "r5", "r2"]
    steps, decode_steps = steps_decode_together(model, rids, tail=12)
    eager = replay(model, dtype, steps, max_tokens=512)
    graphs = {}

    def after(runner):
        graphs["replays"] = runner.graph_replays
    got = replay(model, dtype, steps, max_tokens=512, graphs=True, after=after)
    assert graphs["replays"] == decode_steps
    check(model, dtype, got, "decode graphs")
    if dtype == "float32":
        for key, row in got.items():
            assert torch.equal(row, eager[key]), f"graph replay differs from the eager step at {key}"


def test_greedy_generation_through_the_engine_and_its_scheduler(model):
    """`Engine.generate`: five prompts through three slots and a small pool (queueing, slots and pages used again,
    portions of 16 tokens), 32-bit, against greedy decoding with the plain model."""
    from tensorline_b200 import Engine, SamplingParams
    prompts = [random_tokens(model["vocab"], n, seed=50 + n) for n in (9, 2, 40, 5, 21)]
    want = [greedy_generate(model["plain"], p, 8) for p in prompts]
    for graphs in (False, True):
        eng = Engine(str(model["folder"]), dtype="float32", block_size=model["page"], num_blocks=160 // model["page"], max_num_seqs=3,
                     max_model_len=64, max_batched_tokens=16, cuda_graphs=graphs, overlap=graphs)
        got = [o.token_ids for o in eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
        assert got == want, f"graphs {graphs}: {got} != {want}"
        st = eng.stats()
        assert st["free_pages"] == st["num_pages"] and st["max_running_seen"] == 3 and (st["graph_replays"] > 0) == graphs


@pytest.mark.parametrize("name", ["D3", "D4", "D5"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_further_shapes_of_the_design(name, dtype, tmp_path):
    """The delta rule only (no page group at all, no loop, every expert chosen, grouped heads); a window of one token, a
    latent without a window, a loop of one pass; sizes that are multiples of nothing much and a latent without a rotated
    part: whole requests and changing portions against the plain model."""
    folder = write_tiny_dekerax(name, tmp_path / name)
    plain = PlainDekerax(folder)
    V = CONFIGS[name]["vocab"]
    reqs = {f"r{i}": random_tokens(V, n, seed=300 + i) for i, n in enumerate([3, 50, 1, 81])}
    m = dict(name=name, folder=folder, reqs=reqs, want={r: forward(plain, t) for r, t in reqs.items()}, page=PAGE_SIZE[name], vocab=V)
    whole = replay(m, dtype, steps_alone(m, cuts_whole), max_tokens=128)
    check(m, dtype, whole, "whole")
    cut = replay(m, dtype, steps_alone(m, cuts_changing), max_tokens=128)
    check(m, dtype, cut, "changing portions")
    if dtype == "float32":
        assert all(torch.equal(cut[k], whole[k]) for k in whole)


def test_generate_from_the_command_line(model, capsys):
    """The `tensorline` command with token ids, 32-bit, against greedy decoding with the plain model."""
    from tensorline_b200 import cli
    assert cli.main(["--model", str(model["folder"]), "--dtype", "float32", "--prompt-ids", "5,9,40,17", "--prompt-ids", "7",
                     "--max-tokens", "5", "--ignore-eos", "--block-size", str(model["page"]), "--num-blocks", "16",
                     "--max-num-seqs", "4", "--max-model-len", "64"]) == 0
    import json
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert [l["token_ids"] for l in lines] == [greedy_generate(model["plain"], [5, 9, 40, 17], 5), greedy_generate(model["plain"], [7], 5)]
