"""The kernels of the Lafanex parts on the device, each against the plain formula of tests/plain/lafanex_plain.py: the
residual streams' step, the gate functions, the attention with a sink (both cache layouts, split keys against one block a
token), the selective scan (every lane class, states carried from call to call, a thousand slow decays in a row), routing
with softmax scores, a correction and identity experts, and the weighted combine."""
import math

import pytest
import torch

from tests import helpers as H
from tests.plain import lafanex_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    err = H.scaled_error(got.float(), want)
    print(f"MEASURED {what} {dtype}: {err:.3e}")
    assert err < (f32 if dtype == torch.float32 else bf16), (what, err)


def i32(values):
    return torch.tensor(values, dtype=torch.int32).cuda()


# ------------------------------------------------------------------------------------------------ residual streams
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams,width", [(1, 20), (3, 45), (4, 192), (8, 1024)])
def test_a_step_over_the_residual_streams(kernels, dtype, streams, width):
    g = torch.Generator().manual_seed(streams * width)
    T, S = 7, streams
    r = lambda *shape: torch.randn(*shape, generator=g)
    emb, y = r(T, width).to(dtype), r(T, width).to(dtype)
    read, mix, write, norm_w = r(S) / S, torch.eye(S) + 0.2 * r(S, S), 1 + 0.1 * r(S), 1 + 0.1 * r(width)
    x = torch.empty(T, S, width).cuda()
    first = kernels.stream_step(x, norm_w.cuda(), 1e-5, dtype, read=read.cuda(), init_from=emb.cuda())
    copies = emb.double()[:, None, :].expand(T, S, width)
    assert torch.equal(x.cpu().double(), copies)                       # every stream starts as the embedding
    close(first, P.offset_norm(torch.einsum("s,tsw->tw", read.double(), copies), norm_w.double() - 1, 1e-5), dtype, "first read")
    x0 = (3 * r(T, S, width)).cuda()
    x = x0.clone()
    want_x = torch.einsum("sr,tsw->trw", mix.double(), x0.cpu().double()) + write.double()[None, :, None] * y.double()[:, None, :]
    out = kernels.stream_step(x, norm_w.cuda(), 1e-5, dtype, read=read.cuda(), y=y.cuda(), mix=mix.cuda(), write=write.cuda())
    assert H.scaled_error(x, want_x) < 2e-6                            # the streams stay 32-bit whatever the activation dtype is
    close(out, P.offset_norm(torch.einsum("s,tsw->tw", read.double(), want_x), norm_w.double() - 1, 1e-5), dtype, "write-back and read")
    # the model's end: the write-back is applied but not stored, the streams of the chosen rows are summed
    x = x0.clone()
    rows = i32([5, 0, 5, 2])
    last = kernels.stream_step(x, norm_w.cuda(), 1e-5, dtype, y=y.cuda(), mix=mix.cuda(), write=write.cuda(), rows=rows)
    assert torch.equal(x, x0)
    close(last, P.offset_norm(want_x.sum(1), norm_w.double() - 1, 1e-5)[[5, 0, 5, 2]], dtype, "the sum of the streams of chosen rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("activation,limit", [("silu", 0.0), ("gelu_tanh", 0.0), ("clamped_swish", 1.5)])
def test_gate_functions(kernels, dtype, activation, limit):
    g = torch.Generator().manual_seed(3)
    x = (2.5 * torch.randn(5, 2 * 37, generator=g)).to(dtype)
    gate, up = x[:, :37].double(), x[:, 37:].double()
    if activation == "silu":
        want = P.silu(gate) * up
    elif activation == "gelu_tanh":
        want = P.gelu_tanh(gate) * up
    else:
        gl, ul = torch.clamp(gate, max=limit), torch.clamp(up, min=-limit, max=limit)
        want = gl * torch.sigmoid(1.702 * gl) * (ul + 1)
    close(kernels.gated_act_mul(x.cuda(), activation, limit), want, dtype, f"gate function {activation}")


# ------------------------------------------------------------------------------------------------ attention with a sink
def paged_rows(lengths, page_size, seed):
    """Block tables of requests of the given lengths over shuffled pages: (kv_indptr, kv_indices, number of pages)."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // page_size) for n in lengths]
    perm = torch.randperm(sum(need) + 3, generator=g).tolist()
    indptr, indices = [0], []
    for n in need:
        indices += perm[len(indices) : len(indices) + n]
        indptr.append(len(indices))
    return indptr, indices, sum(need) + 3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot", [(4, 2, 6, 5, 4), (3, 3, 16, 16, 16), (12, 1, 24, 40, 10), (4, 2, 64, 64, 32), (2, 1, 7, 3, 6)])
@pytest.mark.parametrize("sink", [True, False])
def test_attention_with_a_sink_over_pages_against_the_plain_sum(kernels, dtype, heads, kv_heads, dim, vdim, rot, sink):
    """Three requests of unequal length: a whole prompt, a portion whose earlier keys are in the cache already, a single
    decoded token after 70 keys; pages shuffled; both cache layouts (two planes when keys and values have one size); the keys
    dealt to several blocks against one block a token."""
    g = torch.Generator().manual_seed(heads * dim + vdim)
    page_size, eps, scale, base = 4, 1e-5, 0.4 / math.sqrt(dim) * 4, 300.0
    lengths, news = [33, 50, 71], [33, 9, 1]            # tokens a request holds after the step, and how many of them are new
    indptr, indices, pages = paged_rows(lengths, page_size, seed=dim)
    width = (heads + kv_heads) * dim + kv_heads * vdim
    full = [(1.5 * torch.randn(n, width, generator=g)).to(dtype) for n in lengths]       # every token's q | k | v rows
    two_planes = dim == vdim
    if two_planes:
        pool = torch.full((2, pages, kv_heads, page_size, dim), float("nan"), dtype=dtype).cuda()
        k_pool, v_pool = pool[0], pool[1]
    else:
        k_pool, v_pool = torch.full((pages, kv_heads, page_size, dim + vdim), float("nan"), dtype=dtype).cuda(), None
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).cuda()

    def run(rows, kv_cap):
        """rows: (request, first position, count). Prepares and attends the rows' tokens; returns [tokens, heads * vdim]."""
        qkv = torch.cat([full[r][a : a + n] for r, a, n in rows]).cuda()
        positions = i32([p for r, a, n in rows for p in range(a, a + n)])
        token_row = i32([b for b, (r, a, n) in enumerate(rows) for _ in range(n)])
        slots = i32([indices[indptr[r] + p // page_size] * page_size + p % page_size for r, a, n in rows for p in range(a, a + n)])
        kvp, kvi = [0], []
        for r, a, n in rows:
            kvi += indices[indptr[r] : indptr[r + 1]]
            kvp.append(len(kvi))
        kernels.sink_attention_prepare(qkv, k_pool, v_pool, inv_freq, rot, positions, slots, heads, kv_heads, dim, vdim, eps, page_size)
        return kernels.sink_attention(qkv, k_pool, v_pool, positions, token_row, i32(kvp), i32(kvi), heads, kv_heads, dim, vdim, scale, sink,
                                      kv_cap=kv_cap)

    run([(r, 0, lengths[r] - news[r]) for r in (1, 2)], 0)                     # what the cache holds before the step
    rows = [(r, lengths[r] - news[r], news[r]) for r in range(3)]
    one_block = run(rows, 0)
    split = run(rows, 1024)                                                     # a bound on the lengths: the keys are dealt to several blocks
    want = []
    for r in range(3):
        x = full[r].double()
        Q, K = heads * dim, kv_heads * dim
        pos = list(range(lengths[r]))
        q = P.unit_rms(P.rotate_pairs(x[:, :Q].reshape(-1, heads, dim), pos, rot, base), eps)
        k = P.unit_rms(P.rotate_pairs(x[:, Q : Q + K].reshape(-1, kv_heads, dim), pos, rot, base), eps)
        if dtype == torch.bfloat16:      # the cache and the prepared queries are rounded to the activation dtype
            q, k = q.to(dtype).double(), k.to(dtype).double()
        v = x[:, Q + K :].reshape(-1, kv_heads, vdim)
        out = torch.zeros(lengths[r], heads, vdim, dtype=torch.float64)
        for h in range(heads):
            s = (q[:, h] @ k[:, h // (heads // kv_heads)].T) * scale
            e = torch.where(torch.tril(torch.ones_like(s)).bool(), torch.exp(s), torch.zeros_like(s))
            out[:, h] = (e / ((1.0 if sink else 0.0) + e.sum(-1, keepdim=True))) @ v[:, h // (heads // kv_heads)]
        want.append(out.reshape(lengths[r], heads * vdim)[lengths[r] - news[r] :])
    want = torch.cat(want)
    close(one_block, want, dtype, "attention, one block a token")
    close(split, want, dtype, "attention, split keys")


# ------------------------------------------------------------------------------------------------ the selective scan
def plain_scan(xc, dt_raw, dbc, z, dt_bias, a, d, S, R, N):
    """Float64; returns (y * silu(z), final S)."""
    out = torch.zeros_like(xc)
    for t in range(xc.shape[0]):
        dt = P.softplus(dt_raw[t] + dt_bias)
        S = torch.exp(dt[:, None] * a) * S + (dt * xc[t])[:, None] * dbc[t, R : R + N][None, :]
        out[t] = (S @ dbc[t, R + N : R + 2 * N] + d * xc[t]) * P.silu(z[t])
    return out, S


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,state,rank", [(10, 5, 3), (64, 16, 4), (37, 24, 2), (48, 40, 6), (20, 130, 1)])
def test_the_selective_scan_at_every_lane_class_with_states_carried_on(kernels, dtype, inner, state, rank):
    g = torch.Generator().manual_seed(inner + state)
    r = lambda *shape: torch.randn(*shape, generator=g)
    rows = [13, 1, 22]                                   # three requests; the second call brings each some more tokens
    slots = i32([2, 0, 3])
    a = -torch.exp(-2 + 2 * torch.rand(inner, state, generator=g))
    dt_bias, d = -1 + 0.5 * r(inner), 1 + 0.3 * r(inner)
    st = torch.zeros(5, inner * state + 7).cuda()       # slots wider than S: what follows S is not touched
    st[:, inner * state :] = 9.0
    S = [torch.zeros(inner, state, dtype=torch.float64) for _ in rows]
    for call in range(2):
        T = sum(rows)
        xc, dbc, xz, dt_raw = r(T, inner).to(dtype), r(T, rank + 2 * state).to(dtype), r(T, 2 * inner).to(dtype), r(T, inner)
        indptr = [0]
        for n in rows:
            indptr.append(indptr[-1] + n)
        got = kernels.mamba1_scan(xc.cuda(), dt_raw.cuda(), dbc.cuda(), xz.cuda(), dt_bias.cuda(), a.cuda(), d.cuda(), st, i32(indptr), slots,
                                  inner, state, rank)
        want = []
        for b in range(len(rows)):
            lo, hi = indptr[b], indptr[b + 1]
            y, S[b] = plain_scan(xc[lo:hi].double(), dt_raw[lo:hi].double(), dbc[lo:hi].double(), xz[lo:hi, inner:].double(), dt_bias.double(),
                                 a.double(), d.double(), S[b], rank, state)
            want.append(y)
        close(got, torch.cat(want), dtype, f"scan call {call}", f32=5e-5)
        rows = [4, 30, 1]
    for b, slot in enumerate(slots.tolist()):
        assert H.scaled_error(st[slot, : inner * state].reshape(inner, state), S[b]) < 5e-5
    assert bool((st[:, inner * state :] == 9.0).all()) and bool((st[1] == torch.cat([torch.zeros(inner * state), torch.full((7,), 9.0)]).cuda()).all())


def test_a_thousand_slow_decays_in_a_row_do_not_drift(kernels):
    """States that live for thousands of tokens are multiplied by decays just below one at every token: an exponential whose
    error leans one way makes the float32 state drift far beyond what rounding to nearest does."""
    g = torch.Generator().manual_seed(9)
    inner, state, rank, T = 32, 16, 2, 1500
    a = -torch.exp(-1 + torch.rand(inner, state, generator=g))
    dt_bias, d = torch.full((inner,), -6.0), torch.ones(inner)          # dt around 0.0025: decays of 0.997 to 0.999
    xc, dbc, xz, dt_raw = (torch.randn(T, inner, generator=g), torch.randn(T, rank + 2 * state, generator=g), torch.randn(T, 2 * inner, generator=g),
                           0.3 * torch.randn(T, inner, generator=g))
    st = torch.zeros(1, inner * state).cuda()
    got = kernels.mamba1_scan(xc.cuda(), dt_raw.cuda(), dbc.cuda(), xz.cuda(), dt_bias.cuda(), a.cuda(), d.cuda(), st, i32([0, T]), i32([0]), inner,
                              state, rank)
    want, S = plain_scan(xc.double(), dt_raw.double(), dbc.double(), xz[:, inner:].double(), dt_bias.double(), a.double(), d.double(),
                         torch.zeros(inner, state, dtype=torch.float64), rank, state)
    err = float((st[0].reshape(inner, state).double().cpu() - S).abs().max() / S.abs().max())
    print(f"MEASURED state after {T} slow decays: {err:.3e}; outputs {H.scaled_error(got, want):.3e}")
    assert err < 3e-6 and H.scaled_error(got, want) < 1e-5


# ------------------------------------------------------------------------------------------------ routing
@pytest.mark.parametrize("experts,identity,top,extra", [(5, 2, 3, 1), (8, 0, 2, 0), (3, 4, 4, 1), (40, 1, 6, 0)])
def test_softmax_routing_with_a_correction_and_identity_experts(kernels, experts, identity, top, extra):
    g = torch.Generator().manual_seed(experts + top)
    T, H_, routed = 29, 12, experts + identity
    logits = (2 * torch.randn(T, routed + extra, generator=g)).cuda()           # a further column rides along and is not routed
    correction = (0.05 * torch.randn(routed, generator=g)).cuda()
    route = kernels.moe_route(logits, top, score="softmax", correction=correction, scale=2.5, routed=routed, real=experts)
    s = torch.softmax(logits[:, :routed].double().cpu(), -1)
    chosen = torch.topk(s + correction.double().cpu(), top, dim=-1).indices
    inverse, expert, weight, token = route.inverse.cpu().long(), route.expert.cpu().long(), route.weight.cpu().double(), route.token.cpu().long()
    assert torch.equal(expert[inverse].reshape(T, top), chosen)                  # the choices, in order
    assert torch.equal(token[inverse].reshape(T, top), torch.arange(T)[:, None].expand(T, top))
    assert float((weight[inverse].reshape(T, top) - 2.5 * s.gather(1, chosen)).abs().max()) < 1e-6
    assert bool((expert[1:] >= expert[:-1]).all())                               # sorted by expert
    tiles = route.tiles.cpu().reshape(-1, 3)
    tiles = tiles[tiles[:, 0] >= 0]
    assert bool((tiles[:, 0] < experts).all())                                   # identity experts have no tiles
    covered = sum(int(b - a) for _, a, b in tiles.tolist())
    assert covered == int((expert < experts).sum())
    # the weighted combine: an identity expert gives the token's own row back; the shared expert is gated
    for dtype in DTYPES:
        x, ys = torch.randn(T, H_, generator=g).to(dtype), torch.randn(T * top, H_, generator=g).to(dtype)
        shared = torch.randn(T, H_, generator=g).to(dtype)
        rows = torch.where((expert < experts)[:, None], ys.double(), x.double()[token]) * weight[:, None]
        want = rows[inverse].reshape(T, top, H_).sum(1)
        close(kernels.moe_combine_weighted(ys.cuda(), route, x.cuda()), want, dtype, "weighted combine")
        if extra:
            gate = torch.sigmoid(logits[:, -1:].double().cpu())
            close(kernels.moe_combine_weighted(ys.cuda(), route, x.cuda(), shared.cuda(), logits), want + gate * shared.double(), dtype,
                  "weighted combine with a gated shared expert")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,ff", [(5, 24), (90, 40), (700, 128)])
def test_expert_products_with_the_clamped_swish_skip_identity_rows(kernels, dtype, tokens, ff):
    """Few rows (a warp an output), tiles of rows, and in bfloat16 with 1,400 sorted rows and an expert size of 128 the grouped
    tcgen05 product: each against the plain expert."""
    g = torch.Generator().manual_seed(tokens)
    E, I, top, Hd, limit = 4, 2, 2, 64, 1.2
    x = torch.randn(tokens, Hd, generator=g).to(dtype)
    gate, up, down = (0.3 * torch.randn(E, ff, Hd, generator=g)).to(dtype), (0.3 * torch.randn(E, ff, Hd, generator=g)).to(dtype), (0.3 * torch.randn(E, Hd, ff, generator=g)).to(dtype)
    logits = torch.randn(tokens, E + I, generator=g).cuda()
    route = kernels.moe_route(logits, top, score="softmax", scale=1.0, routed=E + I, real=E)
    xs = kernels.moe_gather_scale(x.cuda(), route, scale=False)
    assert torch.equal(xs.cpu(), x[route.token.cpu().long()])
    gate_up = None
    if dtype == torch.bfloat16 and ff % 128 == 0:
        gate_up = torch.stack([gate.reshape(E, ff // 128, 128, Hd), up.reshape(E, ff // 128, 128, Hd)], dim=2).reshape(E, 2 * ff, Hd).contiguous().cuda()
    act = kernels.moe_expert_gate_up(xs, gate.cuda(), up.cuda(), route, gate_up, activation="clamped_swish", limit=limit)
    ys = kernels.moe_expert_down(act, down.cuda(), route)
    expert = route.expert.cpu().long()
    real = expert < E
    w = {}
    for e in range(E):
        w.update({f"e{e}.gate": gate[e].double(), f"e{e}.up": up[e].double(), f"e{e}.down": down[e].double()})
    want = torch.zeros(tokens * top, Hd, dtype=torch.float64)
    for e in range(E):
        sel = expert == e
        want[sel] = P.clamped_expert(xs.cpu().double()[sel], w, f"e{e}.", limit)
    close(ys[real.cuda()], want[real], dtype, "experts with the clamped swish", bf16=4e-2)


# ------------------------------------------------------------------------------------------------ the sink on the tensor cores
@pytest.mark.parametrize("faint", [False, True], ids=["random scores", "faint scores"])
@pytest.mark.parametrize("dim,heads,kv_heads", [(64, 4, 2), (128, 8, 2), (32, 2, 2), (64, 6, 2), (128, 5, 1), (256, 2, 1)])
def test_the_tensor_core_attention_kernels_with_a_sink_against_the_32_bit_kernel(tmp_path, kernels, dim, heads, kv_heads, faint):
    """A one-layer model whose keys and values have one size runs its bfloat16 attention on the framework's tensor-core
    kernels with the sink added at their ends: a prompt of 700 tokens (the tcgen05 or mma.sync prefill), portions, three
    requests decoding side by side beyond 512 keys (split rows merged by clusters or by the merge kernel) and one short one.
    The same steps with that path switched off run the 32-bit kernel; both are held against the plain implementation.
    With random weights the sink's one is lost among hundreds of keys, so a second set of weights makes it count at every
    length: all tokens' embeddings nearly alike and every key the negative of its group's first query, so that every score of
    those heads is near -6 and seven hundred keys weigh about as much as the sink."""
    from roost_b200.engine.executor import StepEntry, StepExecutor
    from tests import lafanex_models as LM
    cfg = LM.config([(LM.attention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, rot=2 if faint else dim // 2, base=10000.0,
                                   scale=(6.0 if faint else 2.0) / dim), None)], width=64, vocab=90, streams=2)
    tensors = LM.draw_tensors(cfg, seed=dim)
    if faint:
        g = torch.Generator().manual_seed(5)
        tensors["embed"] = (torch.randn(64, generator=g)[None, :] + 0.1 * torch.randn(90, 64, generator=g)).to(torch.bfloat16)
        q = tensors["l0.mix.q"].reshape(heads, dim, 64)
        tensors["l0.mix.k"] = (-q[:: heads // kv_heads]).reshape(kv_heads * dim, 64).contiguous()
        tensors["l0.mix.o"] = tensors["l0.mix.o"] * 32          # the attention's output decides the logits
    folder = LM.write_model(tmp_path / "m", cfg, tensors)
    weights = LM.plain_weights(tensors)
    reqs = {"a": H.random_ids(760, 90, 1), "b": H.random_ids(600, 90, 2), "c": H.random_ids(530, 90, 3), "d": H.random_ids(9, 90, 4)}
    results = {}
    for tensor_cores in (True, False):
        model = H.make_model(folder, torch.bfloat16, "gpu")
        if not tensor_cores:
            model.rt.kernels.attention_mma_sink = False
        try:
            ex = StepExecutor(model, page_size=16, num_pages=140, max_requests=4)
            outs = {r: [] for r in reqs}

            def step(entries):
                logits = ex.step([StepEntry(r, list(t), list(range(len(t)))) for r, t in entries])
                at = 0
                for r, t in entries:
                    outs[r].append(logits[at : at + len(t)].float().cpu())
                    at += len(t)

            step([("a", reqs["a"][:700])])
            step([("b", reqs["b"][:300]), ("a", reqs["a"][700:720])])
            step([("b", reqs["b"][300:570]), ("c", reqs["c"][:520]), ("d", reqs["d"][:3])])
            at = {"a": 720, "b": 570, "c": 520, "d": 3}
            for _ in range(6):
                step([(r, reqs[r][at[r] : at[r] + 1]) for r in reqs])
                for r in reqs:
                    at[r] += 1
            results[tensor_cores] = {r: torch.cat(v) for r, v in outs.items()}
        finally:
            if not tensor_cores:
                del model.rt.kernels.attention_mma_sink
        model.rt.kernels.check_device_status()
    for r, ids in reqs.items():
        n = results[True][r].shape[0]
        want = P.forward(cfg, weights, ids[:n])
        for tensor_cores in (True, False):
            rms = H.rms_error(results[tensor_cores][r], want)
            print(f"MEASURED head size {dim} request {r} tensor cores {tensor_cores}: rms error {rms:.3e}")
            assert rms < 0.02, (r, tensor_cores, rms)
        assert H.rms_error(results[True][r], results[False][r]) < 0.02
    if faint:       # the test's own sharpness: without the sink the last position's logits of the longest request are far off
        import copy
        from tests.plain import lafanex_plain as plain
        orig = plain.sink_attention
        try:
            def no_sink(h, w, p, m, eps, positions=None):
                T = h.shape[0]
                qq = plain.unit_rms(plain.rotate_pairs((h @ w[p + "q"].T).reshape(T, heads, dim), list(range(T)), m["rot"]["dims"], m["rot"]["base"]), eps)
                kk = plain.unit_rms(plain.rotate_pairs((h @ w[p + "k"].T).reshape(T, kv_heads, dim), list(range(T)), m["rot"]["dims"], m["rot"]["base"]), eps)
                vv = (h @ w[p + "v"].T).reshape(T, kv_heads, dim)
                out = torch.zeros(T, heads, dim, dtype=torch.float64)
                for hh in range(heads):
                    sc = (qq[:, hh] @ kk[:, hh // (heads // kv_heads)].T) * m["scale"]
                    sc = sc.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
                    out[:, hh] = torch.softmax(sc, -1) @ vv[:, hh // (heads // kv_heads)]
                return out.reshape(T, heads * dim) @ w[p + "o"].T
            plain.sink_attention = no_sink
            without = plain.forward(cfg, weights, reqs["a"][:726])
        finally:
            plain.sink_attention = orig
        want_last = P.forward(cfg, weights, reqs["a"][:726])[-1:]
        moved = H.rms_error(without[-1:], want_last)
        errs = [H.rms_error(results[tc]["a"][-1:], want_last) for tc in (True, False)]
        print(f"MEASURED without the sink the last position's logits move by {moved:.4f}; the kernels' errors there: {errs[0]:.2e}, {errs[1]:.2e}")
        assert moved > 8 * max(errs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inner,state", [(40, 16), (33, 24)])
def test_long_rows_of_the_scan_cut_into_chunks_that_run_side_by_side(kernels, dtype, inner, state):
    """Rows of 300, 1, 129, 128, 0 and 257 tokens on states that are not empty: the chunked form (a walk of every chunk from an
    empty state, a carry from chunk to chunk, a second walk that writes the outputs) against one walk a row and the plain sum;
    the slots end with the same states."""
    g = torch.Generator().manual_seed(inner)
    r = lambda *shape: torch.randn(*shape, generator=g)
    rows, rank = [300, 1, 129, 128, 0, 257], 3
    T = sum(rows)
    indptr = [0]
    for n in rows:
        indptr.append(indptr[-1] + n)
    slots = i32([4, 1, 0, 5, 2, 3])
    a = -torch.exp(-3 + 2 * torch.rand(inner, state, generator=g))
    dt_bias, d = -2 + 0.5 * r(inner), 1 + 0.3 * r(inner)
    xc, dbc, xz, dt_raw = r(T, inner).to(dtype), r(T, rank + 2 * state).to(dtype), r(T, 2 * inner).to(dtype), r(T, inner)
    start = r(6, inner * state)
    states, outs = {}, {}
    for chunked in (False, True):
        st = start.clone().cuda()
        outs[chunked] = kernels.mamba1_scan(xc.cuda(), dt_raw.cuda(), dbc.cuda(), xz.cuda(), dt_bias.cuda(), a.cuda(), d.cuda(), st, i32(indptr), slots,
                                            inner, state, rank, chunked=chunked)
        states[chunked] = st.cpu()
    want, want_states = [], start.double().clone()
    for b, slot in enumerate(slots.tolist()):
        lo, hi = indptr[b], indptr[b + 1]
        y, S = plain_scan(xc[lo:hi].double(), dt_raw[lo:hi].double(), dbc[lo:hi].double(), xz[lo:hi, inner:].double(), dt_bias.double(), a.double(),
                          d.double(), start[slot].double().reshape(inner, state), rank, state)
        want.append(y)
        want_states[slot] = S.reshape(-1)
    want = torch.cat(want)
    for chunked in (False, True):
        close(outs[chunked], want, dtype, f"scan, chunked {chunked}", f32=5e-5)
        assert H.scaled_error(states[chunked], want_states) < 5e-5


# ------------------------------------------------------------------------------------------------ the programs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_tool_on_a_lafanex_folder(tmp_path, dtype):
    """bin/trace_run finds the model by config.json and drives the engine's step function: a request cut into portions beside
    another one, a step in which nothing is wanted, a request that ends and gives its pages and slot back."""
    import json
    import subprocess
    import sys

    import numpy as np

    from tests import lafanex_models as LM
    from tests.conftest import ROOT
    cfg = LM.WIDE
    tensors = LM.draw_tensors(cfg, 8)
    folder = LM.write_model(tmp_path / "model", cfg, tensors)
    a, b = H.random_ids(70, cfg["vocab"], 1), H.random_ids(41, cfg["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[33:69], "want": [35]}, {"id": "b", "tokens": b[2:], "want": [38]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [line for line in r.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert not (out / "1.f32").exists()
    read = lambda n, rows: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(rows, cfg["vocab"]))
    w = LM.plain_weights(tensors)
    wa, wb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    bound = 2e-5 if dtype == "float32" else 0.05
    assert H.rms_error(read(0, 2), wa[[0, 32]]) < bound
    assert H.rms_error(read(2, 2), torch.stack([wa[68], wb[40]])) < bound
    assert H.rms_error(read(3, 1), wa[69:70]) < bound


def test_the_command_line_writes_a_lafanex_folder_and_generates_from_it(tmp_path):
    """random-weights draws the folder from the configuration alone (decay rates, step biases and the streams' weights by their
    declarations' hints), generate runs it through the entry point; the greedy tokens are the plain implementation's wherever
    its choice is clear."""
    import json
    import subprocess
    import sys

    from roost_b200.weights.safetensors_io import SafetensorsFile
    from tests import lafanex_models as LM
    from tests.conftest import ROOT
    roost = lambda *a: subprocess.run([sys.executable, str(ROOT / "bin" / "roost"), *a], capture_output=True, text=True, timeout=600)
    (tmp_path / "config.json").write_text(json.dumps(LM.MIXED))
    r = roost("random-weights", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "model"), "--seed", "4", "--std", "0.1",
              "--norm-std", "0.0")
    assert r.returncode == 0, r.stderr
    f = SafetensorsFile(tmp_path / "model" / "model.safetensors")
    w = {n: f.tensor(n).clone().double() for n in f.names()}
    assert tuple(w["l1.hc2.mix"].shape) == (3, 3) and float((w["l1.hc2.mix"] - torch.eye(3, dtype=torch.float64)).abs().max()) < 0.5
    # the folder's norm weights are drawn around one, as the engine's other models store them; the design adds one to what is stored
    cfg = LM.MIXED
    prompt = H.random_ids(21, cfg["vocab"], 6)
    r = roost("generate", "--model", str(tmp_path / "model"), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
              "--max-output-tokens", "8", "--ignore-eos", "--attention-blocks", "16", "--max-sequences", "2")
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["finish_reason"] == "length" and len(out["token_ids"]) == 8
    logits = P.forward(cfg, w, prompt + out["token_ids"][:-1])
    for j, tok in enumerate(out["token_ids"]):
        top = logits[len(prompt) - 1 + j].topk(2)
        if float(top.values[0] - top.values[1]) > 1e-3:
            assert tok == int(top.indices[0]), (j, tok, int(top.indices[0]))
