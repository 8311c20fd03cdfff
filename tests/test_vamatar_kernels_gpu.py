"""The kernels of the Vamatar parts on the device, each against the plain formula, and the forms a step chooses between
against one another (split keys against one block a token, a warp an output against tiles of rows); sizes of every
register class of the scan kernel; the replay tool on a Vamatar folder."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from roost_b200.engine.executor import StepEntry, StepExecutor
from tests import helpers as H
from tests import vamatar_models as VM
from tests.conftest import ROOT
from tests.plain import vamatar_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    err = H.scaled_error(got.float(), want)
    print(f"MEASURED {what} {dtype}: {err:.3e}")
    assert err < (f32 if dtype == torch.float32 else bf16), (what, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [20, 352, 4096])
def test_layer_norm_over_a_32_bit_stream(kernels, dtype, hidden):
    g = torch.Generator().manual_seed(hidden)
    stream = (torch.randn(9, hidden, generator=g) * 3 + 1).cuda()
    addend = torch.randn(9, hidden, generator=g).to(dtype).cuda()
    w, b = torch.randn(hidden, generator=g).cuda(), torch.randn(hidden, generator=g).cuda()
    want_sum = stream.double().cpu() + addend.double().cpu()
    want = P.layer_norm(want_sum, w.double().cpu(), b.double().cpu(), 1e-5)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
    before = stream.clone()
    gathered = kernels.layer_norm(stream, w, b, 1e-5, dtype, addend, rows)
    assert torch.equal(stream, before)                  # gathered rows leave the stream as it is
    close(gathered, want[[7, 0, 3]], dtype, "layer norm of gathered rows")
    out = kernels.layer_norm(stream, w, b, 1e-5, dtype, addend)
    close(out, want, dtype, "add + layer norm")
    assert H.scaled_error(stream, want_sum) < 1e-6      # the stream holds the 32-bit sum, not a rounded one
    close(kernels.layer_norm(stream, w, b, 1e-5, dtype), want, dtype, "layer norm alone")


def test_scaled_embedding_and_capped_logits(kernels):
    table = torch.randn(30, 24).to(torch.bfloat16).cuda()
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32).cuda()
    out = kernels.embedding_scaled(table, ids, 0.3)
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table.float().cpu()[ids.long().cpu()] * torch.tensor(0.3))
    z = (torch.randn(5, 77) * 30).cuda()
    want = 12.0 * torch.tanh(z.double().cpu() / 12.0)
    assert H.scaled_error(kernels.softcap_(z.clone(), 12.0), want) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 37])
def test_latent_attention_with_split_keys_against_the_plain_sum(kernels, dtype, window):
    """Three rows of unequal length, one token each at the end of 5, 130 and 260 cached entries on pages of 8 handed out in
    a scrambled order; the keys of a token dealt to several blocks (a decode step of few rows) and to one."""
    heads, nope, rope, rank, page = 5, 8, 6, 20, 8
    g = torch.Generator().manual_seed(3)
    lens = [5, 130, 260]
    n_pages = sum(-(-n // page) for n in lens)
    order = torch.randperm(n_pages, generator=g).tolist()
    pool = torch.zeros(n_pages, 1, page, rank + rope)
    entries, tables = [], []
    for n in lens:
        e = torch.randn(n, rank + rope, generator=g)
        mine = [order.pop() for _ in range(-(-n // page))]
        for j in range(n):
            pool[mine[j // page], 0, j % page] = e[j]
        entries.append(e)
        tables.append(mine)
    pool = pool.to(dtype).cuda()
    T = len(lens)
    q_latent = torch.randn(heads, T, rank, generator=g).to(dtype).cuda()
    q = torch.randn(T, heads * (nope + rope), generator=g).to(dtype).cuda()
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    token_row = torch.arange(T, dtype=torch.int32).cuda()
    indptr = torch.tensor([0] + list(np.cumsum([len(t) for t in tables])), dtype=torch.int32).cuda()
    indices = torch.tensor([p for t in tables for p in t], dtype=torch.int32).cuda()
    scale = 0.21
    want = torch.zeros(heads, T, rank, dtype=torch.float64)
    for t, n in enumerate(lens):
        lo = 0 if window is None else max(0, n - window)
        e = pool[:, 0].reshape(-1, rank + rope).double().cpu()
        rows = torch.stack([e[tables[t][j // page] * page + j % page] for j in range(lo, n)])
        qr = q[t].double().cpu().reshape(heads, nope + rope)[:, nope:]
        s = (q_latent[:, t].double().cpu() @ rows[:, :rank].T + qr @ rows[:, rank:].T) * scale
        want[:, t] = torch.softmax(s, -1) @ rows[:, :rank]
    args = (q_latent, q, pool, positions, token_row, indptr, indices, heads, nope, rope, rank, scale, window)
    one = kernels.latent_attention(*args, 0)
    split = kernels.latent_attention(*args, 1024, True)
    assert kernels.latent_splits_for(T, heads, window, 1024) > 1
    close(one, want, dtype, "latent attention, one block a token", bf16=1e-2)
    close(split, want, dtype, "latent attention, split keys", bf16=1e-2)


@pytest.mark.parametrize("rank", [32, 80, 272])
@pytest.mark.parametrize("window", [None, 37])
def test_latent_attention_on_the_tensor_cores_against_the_plain_sum(kernels, rank, window):
    """Portions of three requests in one step (77 tokens after 60 cached ones, 5 from the start, 140 after 3), five heads, so
    that the packed (token, head) rows of a tile span several tokens with windows of their own; pages of 8 in a scrambled
    order; with a window the pages it has passed are gone from the block tables (-1)."""
    heads, nope, rope, page = 5, 8, 8, 8
    g = torch.Generator().manual_seed(rank)
    spans = [(60, 77), (0, 5), (3, 140)]
    totals = [a + n for a, n in spans]
    n_pages = sum(-(-n // page) for n in totals)
    order = torch.randperm(n_pages, generator=g).tolist()
    pool = torch.zeros(n_pages, 1, page, rank + rope)
    tables, entries = [], []
    for (start, n), total in zip(spans, totals):
        e = torch.randn(total, rank + rope, generator=g)
        mine = [order.pop() for _ in range(-(-total // page))]
        for j in range(total):
            pool[mine[j // page], 0, j % page] = e[j]
        if window:            # pages wholly before the first query's window are given back
            for i in range(max(0, start - window + 1) // page):
                pool[mine[i]] = float("nan")
                mine[i] = -1
        entries.append(e)
        tables.append(mine)
    pool = pool.to(torch.bfloat16).cuda()
    T = sum(n for _, n in spans)
    q_latent = torch.randn(heads, T, rank, generator=g)
    if window:
        # two queries of the first request made to score one key far above the rest: the oldest key its window keeps (position
        # 100 sees 64..100), and the first key its window has dropped (position 110 sees 74..110, not 73); a window one off
        # turns either result into another
        q_latent[:, 40] = 2.0 * entries[0][100 - window + 1, :rank]
        q_latent[:, 50] = 2.0 * entries[0][110 - window, :rank]
    q_latent = q_latent.to(torch.bfloat16).cuda()
    q = torch.randn(T, heads * (nope + rope), generator=g).to(torch.bfloat16).cuda()
    positions = torch.tensor([start + i for start, n in spans for i in range(n)], dtype=torch.int32).cuda()
    token_row = torch.tensor([b for b, (_, n) in enumerate(spans) for _ in range(n)], dtype=torch.int32).cuda()
    q_indptr = torch.tensor([0] + list(np.cumsum([n for _, n in spans])), dtype=torch.int32).cuda()
    indptr = torch.tensor([0] + list(np.cumsum([len(t) for t in tables])), dtype=torch.int32).cuda()
    indices = torch.tensor([p for t in tables for p in t], dtype=torch.int32).cuda()
    scale = 0.3
    want = torch.zeros(heads, T, rank, dtype=torch.float64)
    t = 0
    for b, (start, n) in enumerate(spans):
        e = entries[b].to(torch.bfloat16).double()
        for i in range(n):
            pos = start + i
            lo = 0 if window is None else max(0, pos - window + 1)
            rows = e[lo : pos + 1]
            qr = q[t].double().cpu().reshape(heads, nope + rope)[:, nope:]
            sc = (q_latent[:, t].double().cpu() @ rows[:, :rank].T + qr @ rows[:, rank:].T) * scale
            want[:, t] = torch.softmax(sc, -1) @ rows[:, :rank]
            t += 1
    got = kernels.latent_attention(q_latent, q, pool, positions, token_row, indptr, indices, heads, nope, rope, rank, scale, window, 1024,
                                   False, q_indptr)
    assert kernels._lib.roost_latent_attention_tc_supported(nope, rope, rank) and T * heads >= kernels.LATENT_TC_MIN_ROWS
    close(got, want, torch.bfloat16, f"latent attention on the tensor cores, rank {rank}", bf16=1.5e-2)
    slow = kernels.latent_attention(q_latent, q, pool, positions, token_row, indptr, indices, heads, nope, rope, rank, scale, window, 0)
    close(slow, want, torch.bfloat16, "the 32-bit form on the same step", bf16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_routing_chooses_the_largest_scores_and_sorts_the_pairs_by_expert(kernels, dtype):
    T, E, top, hidden, ff = 50, 9, 3, 24, 16
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(T, E, generator=g) * 3
    logits[4, 2] = logits[4, 6] = logits[4].max() + 1          # a tie goes to the lower index
    route = kernels.moe_route(logits.cuda(), top)
    token, expert, weight, inverse = route.token.cpu(), route.expert.cpu(), route.weight.cpu(), route.inverse.cpu().long()
    assert torch.equal(expert, expert.sort().values)            # sorted by expert
    offsets = route.offsets.cpu()
    assert int(offsets[-1]) == T * top and all(int((expert == e).sum()) == int(offsets[e + 1] - offsets[e]) for e in range(E))
    for t in range(T):
        want = sorted(range(E), key=lambda e: (-float(logits[t, e]), e))[:top]
        assert [int(expert[inverse[t * top + k]]) for k in range(top)] == want
        assert all(int(token[inverse[t * top + k]]) == t for k in range(top))
        for k, e in enumerate(want):
            assert abs(float(weight[inverse[t * top + k]]) - float(torch.sigmoid(logits[t, e].double()))) < 1e-6
    tiles = route.tiles.cpu().reshape(-1, 3)
    covered = sorted((int(a), int(b)) for e, a, b in tiles if e >= 0)
    assert covered[0][0] == 0 and covered[-1][1] == T * top and all(x[1] == y[0] for x, y in zip(covered, covered[1:]))
    # the expert products in both forms, and the sum
    x = torch.randn(T, hidden, generator=g).to(dtype).cuda()
    wg, wu = (torch.randn(E, ff, hidden, generator=g) * 0.3).to(dtype).cuda(), (torch.randn(E, ff, hidden, generator=g) * 0.3).to(dtype).cuda()
    wd = (torch.randn(E, hidden, ff, generator=g) * 0.3).to(dtype).cuda()
    shared = torch.randn(T, hidden, generator=g).to(dtype).cuda()
    xs = kernels.moe_gather_scale(x, route)
    outs = []
    for form in (0, 1):
        a = torch.empty(T * top, ff, dtype=dtype, device="cuda")
        kernels._call("roost_moe_expert_gemm", xs.data_ptr(), wg.data_ptr(), wu.data_ptr(), a.data_ptr(), route.tiles.data_ptr(), route.max_tiles,
                      route.expert.data_ptr(), T * top, ff, hidden, form, 0, 0, 0.0, 1 << 30, 0 if dtype == torch.float32 else 1, torch.cuda.current_stream().cuda_stream)
        y = torch.empty(T * top, hidden, dtype=dtype, device="cuda")
        kernels._call("roost_moe_expert_gemm", a.data_ptr(), wd.data_ptr(), None, y.data_ptr(), route.tiles.data_ptr(), route.max_tiles,
                      route.expert.data_ptr(), T * top, hidden, ff, form, 0, 0, 0.0, 1 << 30, 0 if dtype == torch.float32 else 1, torch.cuda.current_stream().cuda_stream)
        outs.append(kernels.moe_combine(y, route, shared))
    want = shared.double().cpu().clone()
    xd = x.double().cpu()
    for t in range(T):
        for e in sorted(range(E), key=lambda e: (-float(logits[t, e]), e))[:top]:
            xin = (torch.sigmoid(logits[t, e].double()) * xd[t])[None]
            w = {"gate": wg[e].double().cpu(), "up": wu[e].double().cpu(), "down": wd[e].double().cpu()}
            want[t] += P.gated_ff(xin, w, "")[0]
    close(outs[0], want, dtype, "experts on tiles of rows", bf16=4e-2)
    close(outs[1], want, dtype, "experts, a warp an output", bf16=4e-2)


def test_experts_on_tcgen05_for_steps_of_many_rows(kernels):
    """1,230 sorted rows over 9 experts of unequal load (one expert gets no row at all): the grouped tcgen05 product with the
    activation on its accumulator, and the down product, against the tiles on mma.sync and against the plain formula."""
    from roost_b200.kernels.library import MOE_TCGEN05_MIN_ROWS
    T, E, top, hidden, ff = 410, 9, 3, 192, 256
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(T, E, generator=g) * 2
    logits[:, 4] = -50.0                                    # nobody chooses expert 4
    logits[:200, 7] += 6.0                                  # and many choose expert 7: several tiles of one expert
    route = kernels.moe_route(logits.cuda(), top)
    assert T * top >= MOE_TCGEN05_MIN_ROWS and route.wide_tiles is not None
    x = torch.randn(T, hidden, generator=g).to(torch.bfloat16).cuda()
    wg = (torch.randn(E, ff, hidden, generator=g) * 0.15).to(torch.bfloat16).cuda()
    wu = (torch.randn(E, ff, hidden, generator=g) * 0.15).to(torch.bfloat16).cuda()
    wd = (torch.randn(E, hidden, ff, generator=g) * 0.15).to(torch.bfloat16).cuda()
    gate_up = torch.stack([wg.reshape(E, ff // 128, 128, hidden), wu.reshape(E, ff // 128, 128, hidden)], dim=2).reshape(E, 2 * ff, hidden).contiguous()
    xs = kernels.moe_gather_scale(x, route)
    act_tc = kernels.moe_expert_gate_up(xs, wg, wu, route, gate_up)
    act_mma = kernels._moe_gemm(xs, wg, wu, route)
    assert H.scaled_error(act_tc.float(), act_mma.double().cpu()) < 2e-2
    # the interleaved tensor read by the other forms: tiles on mma.sync, tiles on FFMA, a warp an output (few rows)
    assert torch.equal(kernels._moe_gemm(xs, gate_up, None, route, block=128), act_mma)
    few = kernels.moe_route(logits[:10].cuda(), top)
    xs_few = kernels.moe_gather_scale(x[:10], few)
    assert H.scaled_error(kernels._moe_gemm(xs_few, gate_up, None, few, block=128).float(), kernels._moe_gemm(xs_few, wg, wu, few).double().cpu()) < 1e-6
    f32 = lambda t: t.float()
    assert H.scaled_error(kernels._moe_gemm(f32(xs_few), f32(gate_up), None, few, block=128), kernels._moe_gemm(f32(xs_few), f32(wg), f32(wu), few).double().cpu()) < 1e-6
    y_tc = kernels.moe_expert_down(act_mma, wd, route)
    y_mma = kernels._moe_gemm(act_mma, wd, None, route)
    assert H.scaled_error(y_tc.float(), y_mma.double().cpu()) < 2e-2
    kernels.check_device_status()
    expert, xs_c = route.expert.cpu(), xs.double().cpu()
    for row in (0, 1, 127, 128, 129, 700, T * top - 1):
        e = int(expert[row])
        w = {"gate": wg[e].double().cpu(), "up": wu[e].double().cpu(), "down": wd[e].double().cpu()}
        gv, uv = xs_c[row] @ w["gate"].T, xs_c[row] @ w["up"].T
        assert H.scaled_error(act_tc[row].float(), P.silu(gv) * uv) < 2e-2, row


@pytest.mark.parametrize("state,vdim", [(100, 24), (200, 40), (3, 128)])
def test_the_recurrence_at_sizes_of_every_register_class(tmp_path, state, vdim):
    cfg = VM.config([(VM.mamba(heads=2, vdim=vdim, state=state, groups=2, conv=4, norm_groups=1), None)], width=48, vocab=31, cap=None)
    tensors = VM.draw_tensors(cfg, state)
    folder = VM.write_model(tmp_path, cfg, tensors)
    model = H.make_model(folder, torch.float32, "gpu")
    ex = StepExecutor(model, page_size=4, num_pages=8, max_requests=2)
    ids = H.random_ids(45, cfg["vocab"], 1)
    got = torch.cat([ex.step([StepEntry("r", ids[:20], list(range(20)))]), ex.step([StepEntry("r", ids[20:22], [0, 1])])] +
                    [ex.step([StepEntry("r", [t], [0])]) for t in ids[22:]])
    want = P.forward(cfg, VM.plain_weights(tensors), ids)
    assert H.scaled_error(got, want) < 2e-4 and H.rms_error(got, want) < 3e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_rows_cut_into_chunks_that_run_side_by_side(tmp_path, kernels, dtype):
    """A step of 700 + 41 + 130 tokens (three requests, the second and third continuing earlier portions) is long enough for
    the recurrence to cut its rows into chunks: the states the chunks start from, the carried state of each request and the
    decoding that follows must be those of a walk token by token."""
    cfg = VM.config([(VM.mamba(heads=4, vdim=32, state=64, groups=2, conv=4, norm_groups=2), None),
                     (VM.mamba(heads=2, vdim=16, state=16, groups=1, conv=3, norm_groups=1), VM.dense(ff=32))], width=64, vocab=90, cap=None)
    tensors = VM.draw_tensors(cfg, 31)
    folder = VM.write_model(tmp_path, cfg, tensors)
    model = H.make_model(folder, dtype, "gpu")
    ex = StepExecutor(model, page_size=16, num_pages=8, max_requests=3)
    a, b, c = H.random_ids(703, cfg["vocab"], 1), H.random_ids(60, cfg["vocab"], 2), H.random_ids(140, cfg["vocab"], 3)
    assert sum(map(len, (a[:700], b[16:57], c[7:137]))) >= kernels.SCAN_CHUNKED_MIN_TOKENS
    ex.step([StepEntry("b", b[:16], []), StepEntry("c", c[:7], [])])
    out = ex.step([StepEntry("a", a[:700], [0, 127, 128, 699]), StepEntry("b", b[16:57], [40]), StepEntry("c", c[7:137], [0, 129])])
    tail = [ex.step([StepEntry("a", [a[700 + i]], [0]), StepEntry("b", [b[57 + i]], [0]), StepEntry("c", [c[137 + i]], [0])]) for i in range(3)]
    w = VM.plain_weights(tensors)
    wa, wb, wc = P.forward(cfg, w, a), P.forward(cfg, w, b), P.forward(cfg, w, c)
    want = torch.cat([wa[[0, 127, 128, 699]], wb[[56]], wc[[7, 136]]] + [torch.stack([wa[700 + i], wb[57 + i], wc[137 + i]]) for i in range(3)])
    got = torch.cat([out] + tail)
    err, rms = H.scaled_error(got, want), H.rms_error(got, want)
    print(f"MEASURED chunked recurrence {dtype}: worst {err:.3e}, rms {rms:.3e}")
    assert (err < 1e-4 and rms < 1e-5) if dtype == torch.float32 else (err < 0.25 and rms < 0.04)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_tool_on_a_vamatar_folder(tmp_path, dtype):
    cfg = VM.WIDE
    tensors = VM.draw_tensors(cfg, 8)
    folder = VM.write_model(tmp_path / "model", cfg, tensors)
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
    w = VM.plain_weights(tensors)
    wa, wb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    bound = 2e-4 if dtype == "float32" else 0.25
    assert H.scaled_error(read(0, 2), wa[[0, 32]]) < bound
    assert H.scaled_error(read(2, 2), torch.stack([wa[68], wb[40]])) < bound
    assert H.scaled_error(read(3, 1), wa[69:70]) < bound


def test_the_command_line_writes_a_vamatar_folder_and_generates_from_it(tmp_path):
    """random-weights draws the folder from the configuration alone (decay rates and step biases by their declarations' hints),
    generate runs it through the entry point; the greedy tokens are the plain implementation's wherever its choice is clear."""
    roost = lambda *a: subprocess.run([sys.executable, str(ROOT / "bin" / "roost"), *a], capture_output=True, text=True, timeout=600)
    (tmp_path / "config.json").write_text(json.dumps(VM.MIXED))
    r = roost("random-weights", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "model"), "--seed", "4", "--std", "0.2",
              "--norm-std", "0.1")
    assert r.returncode == 0, r.stderr
    cfg, w = P.load_model_dir(tmp_path / "model")
    assert -3.0 <= float(w["l1.mix.A_log"].min()) and float(w["l1.mix.A_log"].max()) <= -0.5
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
