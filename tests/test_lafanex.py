"""The Lafanex decoder through the engine's step function, cache manager, scheduler and entry point, against the plain
implementation of tests/plain/lafanex_plain.py, for every way of cutting the work.

Each test runs on the GPU with the real kernel library in float32 (captured steps) and bfloat16 (marked gpu), and on the
CPU with the stand-in kernels of tests/fake_kernels.py, which checks the host side. In bfloat16 the engine's routing
choices are recorded and handed to the plain implementation, which checks that each was within a rounding of the best
(two nearly equal scores may be ordered differently in lower precision); float32 runs choose for themselves.
"""
import copy
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.config.lafanex import LafanexConfig
from roost_b200.config.reader import ConfigError, ConfigReader
from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.loader import WeightError
from tests import helpers as H
from tests import lafanex_models as LM
from tests.plain import lafanex_plain as P

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]
# Two bounds: the root-mean-square error of all logits of a request, and the largest root-mean-square error of one position's
# logits (both relative to the logits' own root mean square). A fault that strikes one position (a lost key, a wrong page or
# slot in one step) moves that position's logits by tens of percent and barely shows among hundreds of positions; rounding
# alone stays far below both bounds (measured: float32 5e-6 and 3e-5, bfloat16 0.01 to 0.05 and up to 0.15).
F32_TOKEN, F32_RMS = 1e-3, 2e-5
BF16_TOKEN, BF16_RMS = 0.3, 0.06
ROUTE_SLACK = 0.35                   # in choice scores (softmax scores plus the correction): what bfloat16 inputs may move a score by


@pytest.fixture(params=BACKENDS)
def backend(request):
    return request.param


_MODELS: dict = {}


def model_dir(tmp_path_factory, name, cfg, seed, change=None):
    """A model folder written once a session; ``change(cfg, tensors)`` edits the drawn weights first."""
    if name not in _MODELS:
        tensors = LM.draw_tensors(cfg, seed)
        if change is not None:
            change(cfg, tensors)
        _MODELS[name] = (LM.write_model(tmp_path_factory.mktemp(f"lafanex_{name}"), cfg, tensors), cfg, LM.plain_weights(tensors))
    return _MODELS[name]


class Run:
    """Drives a StepExecutor and keeps, per request, the logits of every position and (when recording) the experts the
    engine chose in every routed layer run."""

    def __init__(self, model_dir, cfg, backend, page_size=4, num_pages=64, slots=4):
        kind, self.dtype = backend
        self.cfg = cfg
        self.model = H.make_model(model_dir, self.dtype, kind)
        # bfloat16 steps run uncaptured so that the routing recorder sees every call; float32 steps replay graphs
        self.record = self.dtype == torch.bfloat16
        self.ex = StepExecutor(self.model, page_size=page_size, num_pages=num_pages, max_requests=slots, use_graphs=not self.record)
        self.routed = LM.routed_runs(cfg)
        self.logits: dict = {}
        self.forced: dict = {}

    def step(self, entries):
        """entries: [(request id, tokens)]; every position's logits are asked for."""
        step_entries = [StepEntry(rid, list(toks), list(range(len(toks)))) for rid, toks in entries]
        if self.record:
            with LM.RouteRecorder(self.model.rt.kernels) as rec:
                out = self.ex.step(step_entries)
            assert len(rec.calls) == len(self.routed)
        else:
            out = self.ex.step(step_entries)
        at = 0
        for rid, toks in entries:
            n = len(toks)
            self.logits.setdefault(rid, []).append(out[at : at + n].float().cpu())
            if self.record:
                for run, call in zip(self.routed, rec.calls):
                    self.forced.setdefault(rid, {}).setdefault(run, []).append(call[at : at + n])
            at += n
        self.ex.cache.check_invariants()

    def finish(self, rid):
        self.ex.finish(rid)

    def check(self, rid, ids, weights, what, bf16_bounds=(BF16_TOKEN, BF16_RMS), slack=ROUTE_SLACK, f32_bounds=(F32_TOKEN, F32_RMS)):
        got = torch.cat(self.logits.pop(rid))
        forced = {run: torch.cat(v) for run, v in self.forced.pop(rid, {}).items()} if self.record else None
        n = got.shape[0]
        want = P.forward(self.cfg, weights, list(ids[:n]), forced=forced, slack=slack)
        err, rms = token_error(got, want), H.rms_error(got, want)
        print(f"MEASURED {what} {self.dtype}: worst position's error {err:.3e}, rms error {rms:.3e}")
        worst, bound = f32_bounds if self.dtype == torch.float32 else bf16_bounds
        assert err < worst and rms < bound, f"{what}: worst position's error {err}, rms error {rms}"
        return got, want

    def all_free(self):
        return all(p.used_count == 0 for p in self.ex.cache.pools)


def token_error(got, want) -> float:
    """The largest error of one position: root mean square of its logits' differences over that of its logits."""
    got, want = got.double().cpu(), want.double().cpu()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()).max())


def ids_for(cfg, n, seed):
    return H.random_ids(n, cfg["vocab"], seed)


SINGLE = {
    "attention_only": LM.config([(LM.attention(heads=2, kv_heads=2, dim=6, vdim=5, rot=6), None)], width=24, vocab=50, streams=2),
    "scan_only": LM.config([(LM.mamba(inner=14, state=6, dt_rank=2, conv=4), None)], width=20, vocab=45, streams=4),
    "dense_after_attention": LM.config([(LM.attention(), LM.dense(ff=17))], width=28, vocab=33, streams=None),
    "experts_after_scan": LM.config([(LM.mamba(), LM.moe(experts=6, identity=1, top=2, ff=9, shared=11))], width=32, vocab=40, streams=2),
    # more choices than experts with weights: at least two of a token's four choices are identity experts
    "mostly_identity": LM.config([(LM.attention(heads=2, kv_heads=1, dim=8, vdim=8, rot=4), LM.moe(experts=2, identity=3, top=4, ff=10, shared=0))], width=24, vocab=41,
                                 streams=3),
    "looped_pair": LM.config([(LM.attention(heads=2, kv_heads=1, dim=4, vdim=4, rot=2), None), (LM.mamba(inner=8, state=3, dt_rank=1, conv=2), None)],
                             width=16, vocab=30, streams=2, loop=(0, 2, 3)),
}
ALL = dict(LM.CONFIGS, **SINGLE)


@pytest.fixture(params=sorted(ALL))
def any_model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, ALL[request.param], seed=len(request.param))


@pytest.fixture(params=sorted(LM.CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, LM.CONFIGS[request.param], seed=len(request.param))


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("length", [1, 2, 3, 37, 150])
def test_each_mechanism_and_each_model_on_whole_prompts(any_model, backend, length):
    """Models of one mechanism each (the attention alone, the scan alone, each feed-forward, a looped pair of layers) and the
    mixed models; the shortest prompts are the first tokens of a sequence: the convolution's zeros before the start, an empty
    state, a softmax over one key and the sink."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, length, seed=length)
    run.step([("r", ids)])
    run.finish("r")
    run.check("r", ids, weights, f"{name} whole {length}")
    assert run.all_free()


def test_prefill_against_token_by_token_decoding(model, backend):
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 70, seed=5)
    for head in (0, 1, 38):     # from the very first token on; after one token; after a prompt that ends inside a page
        rid = f"r{head}"
        if head:
            run.step([(rid, ids[:head])])
        for t in ids[head:]:
            run.step([(rid, [t])])
        run.finish(rid)
        run.check(rid, ids, weights, f"{name} decoded from {head}")
    assert run.all_free()


@pytest.mark.parametrize("sizes", [[2, 3, 2, 5, 7, 16, 33], [33, 2, 2, 1, 9], [1, 2]])
def test_portions_of_several_sizes_down_to_two_tokens(model, backend, sizes):
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 90 if len(sizes) > 2 else 25, seed=sum(sizes))
    at, i = 0, 0
    while at < len(ids):
        n = min(sizes[i % len(sizes)], len(ids) - at)
        run.step([("r", ids[at : at + n])])
        at, i = at + n, i + 1
    run.finish("r")
    run.check("r", ids, weights, f"{name} portions {sizes}")


def test_batches_of_unequal_requests_with_pages_and_slots_used_again(model, backend):
    """Six requests of unequal length through three state slots and a pool of pages that holds three of them: portions
    of some beside single tokens of others; a request that ends gives its pages and slot to the next one."""
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=48, slots=3)
    rng = random.Random(11)
    reqs = {f"q{i}": ids_for(cfg, n, seed=20 + i) for i, n in enumerate([41, 9, 64, 23, 2, 55])}
    waiting, live = list(reqs), {}
    slots_seen = set()
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for rid in [r for r in live if rng.random() < 0.8] or [next(iter(live))]:
            left = len(reqs[rid]) - live[rid]
            n = 1 if left <= 6 else min(left - 6, rng.choice([2, 3, 5, 8, 17]))
            entries.append((rid, reqs[rid][live[rid] : live[rid] + n]))
            live[rid] += n
        run.step(entries)
        for gi, g in enumerate(run.ex.groups):
            if g.kind == "state" and g.runs:
                slots_seen.update(run.ex.cache.get(rid).slots[gi] for rid, _ in entries)
        for rid, _ in entries:
            if live[rid] == len(reqs[rid]):
                run.finish(rid)
                del live[rid]
    assert slots_seen <= {0, 1, 2}
    for rid, ids in reqs.items():
        run.check(rid, ids, weights, f"{name} mixed {rid}")
    assert run.all_free()


def test_long_decoding_over_many_pages(model, backend):
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=80)
    ids = ids_for(cfg, 230, seed=3)
    run.step([("r", ids[:3])])
    for t in ids[3:]:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} long decoding")


LONG = LM.config([(LM.attention(heads=4, kv_heads=2, dim=16, vdim=24, rot=8, base=10000.0, scale=0.25), LM.moe(experts=5, identity=1, top=2, ff=128, shared=40)),
                  (LM.mamba(inner=48, state=16, dt_rank=4, conv=4), LM.moe(experts=3, identity=0, top=2, ff=256, shared=0))],
                 width=72, vocab=83, streams=2)


def test_a_long_prompt_takes_the_forms_of_steps_of_many_rows(tmp_path_factory, backend):
    """600 tokens in one step and then 2 + 1: on the device in bfloat16 the experts' products run on the grouped tcgen05
    kernel (1,200 sorted rows, an expert size that is a multiple of 128, a width of 72 that is no multiple of its 64-wide
    k blocks); the other backends take their own forms of the same step."""
    folder, cfg, weights = model_dir(tmp_path_factory, "long", LONG, seed=21)
    run = Run(folder, cfg, backend, page_size=16, num_pages=48)
    ids = ids_for(cfg, 603, seed=8)
    run.step([("r", ids[:600])])
    run.step([("r", ids[600:602])])
    run.step([("r", ids[602:])])
    run.finish("r")
    run.check("r", ids, weights, "long prompt")


# ------------------------------------------------------------------------------------------------ keys that must be seen
FAR = LM.config([(LM.attention(heads=2, kv_heads=1, dim=8, vdim=6, rot=2, scale=1.0), None), (LM.mamba(), LM.dense(ff=16))], width=32, vocab=53, streams=2)
KEY, QUERY = 7, 11        # token ids: QUERY scores KEY far above every other key in the first layer


def sharpened(tmp_path_factory, name, cfg):
    return model_dir(tmp_path_factory, name, cfg, seed=77, change=lambda c, t: LM.sharpen(c, t, KEY, QUERY))


def filler(cfg, n, seed):
    rng = random.Random(seed)
    return [rng.choice([t for t in range(cfg["vocab"]) if t not in (KEY, QUERY)]) for _ in range(n)]


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
def test_a_key_far_away_among_hundreds_at_every_page_offset(tmp_path_factory, backend, decoded):
    """The key token sits 310 to 320 places before the query token, once at every offset of a page of four and across the
    borders of the 32-key tiles; the sharpened weights put nearly all of the query's attention on it, so losing that one key
    (a wrong page, a tile's edge, a split's edge) changes the query's logits by far more than the bound. The test checks its
    own sharpness: without the key token the plain logits of the query's position move by much more than the bound."""
    folder, cfg, weights = sharpened(tmp_path_factory, "far", FAR)
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    seen = {}
    for at in (None, 0, 1, 2, 3, 31, 32, 33):
        ids = filler(cfg, 330, seed=4)
        if at is not None:
            ids[at] = KEY
        ids[321] = QUERY
        rid = f"far{at}"
        if decoded:
            run.step([(rid, ids[:300])])
            for t in ids[300:]:
                run.step([(rid, [t])])
        else:
            run.step([(rid, ids[:130])])
            run.step([(rid, ids[130:])])
        run.finish(rid)
        got, want = run.check(rid, ids, weights, f"far key at {at}")
        seen[at] = want[321]
    for at in (0, 1, 2, 3, 31, 32, 33):
        moved = H.rms_error(seen[at][None], seen[None][None])
        print(f"MEASURED the key at {at} moves the query's logits by {moved:.3f}")
        assert moved > 2 * BF16_TOKEN


def test_the_first_tokens_of_a_sequence_one_by_one(any_model, backend):
    """A request decoded from its very first token: one key and the sink, an empty state, zeros before the convolution."""
    name, folder, cfg, weights = any_model
    run = Run(folder, cfg, backend)
    ids = ids_for(cfg, 6, seed=1)
    for t in ids:
        run.step([("r", [t])])
    run.finish("r")
    run.check("r", ids, weights, f"{name} first tokens")


# ------------------------------------------------------------------------------------------------ the entry point
def test_greedy_generation_through_the_entry_point_and_scheduler(model, backend):
    name, folder, cfg, weights = model
    kind, dtype = backend
    m = H.make_model(folder, dtype, kind)
    engine = RoostEngine(m, page_size=4, attention_blocks=60, max_sequences=3, max_tokens=24, **({"device": "cpu"} if kind == "fake" else {}))
    prompts = [ids_for(cfg, n, seed=60 + n) for n in (19, 5, 31, 2)]
    outs = engine.generate(prompts, GenerationOptions(max_output_tokens=10))
    for p, out in zip(prompts, outs):
        assert out.finish_reason == "length" and len(out.token_ids) == 10
        if dtype != torch.float32:
            continue          # a bfloat16 engine may route a near-tie differently; its logits are checked above
        logits = P.forward(cfg, weights, list(p) + out.token_ids[:-1])
        for j, tok in enumerate(out.token_ids):
            top = logits[len(p) - 1 + j].topk(2)
            if float(top.values[0] - top.values[1]) > 1e-3:
                assert tok == int(top.indices[0]), (j, tok, int(top.indices[0]))
    assert all(pool.used_count == 0 for pool in engine.executor.cache.pools)


# ------------------------------------------------------------------------------------------------ configuration and weights
def test_the_configuration_is_read_by_its_own_keys_and_refuses_what_it_cannot_be():
    cfg = LafanexConfig.from_dict(LM.MIXED)
    spec = cfg.to_spec()
    assert spec.architecture == "Lafanex" and len(spec.blocks) == 4 and spec.tie_embeddings
    assert [e.block for e in spec.schedule] == [0, 1, 2, 1, 2, 3] and all(e.reads_cache_of is None for e in spec.schedule)
    assert spec.blocks[0].connection.streams == 3 and spec.blocks[0].connection.learned
    assert spec.blocks[3].feed_forward is None and spec.blocks[3].post_mixer_norm is None
    assert spec.blocks[0].input_norm.weight_offset == 1.0 and spec.final_norm.weight_offset == 1.0
    ff = spec.blocks[1].feed_forward
    assert (ff.experts, ff.identity_experts, ff.top, ff.route_scale, ff.limit, ff.shared_limit, ff.shared_gate) == (5, 2, 3, 1.7, 2.0, 1.5, True)
    assert spec.blocks[2].feed_forward.shared_gate is False and spec.blocks[0].feed_forward.activation == "gelu_tanh"
    a = spec.blocks[2].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.v_dim, a.position.rotary_dim, a.position.kind) == (3, 1, 6, 9, 6, "rope_interleaved")
    plain = LafanexConfig.from_dict(LM.PLAIN).to_spec()
    assert plain.blocks[0].connection.streams == 1 and not plain.blocks[0].connection.learned
    assert [e.block for e in plain.schedule] == [0, 1, 0, 1]
    assert "blocks.0.mixer_connection" not in plain.weight_names

    def broken(path, value):
        c = copy.deepcopy(LM.MIXED)
        node = c
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return c

    for path, value, word in [(("layers", 1, "type"), "lstm", "type"), (("layers", 1, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 1, "mlp", "router", "top"), 9, "top"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("norm",), None, "norm.eps"), (("width",), 0, "width"), (("layers", 0, "mixer", "rot", "dims"), 3, "dims"),
                              (("loop", "stop"), 7, "stop"), (("layers", 1, "mlp", "expert", "limit"), 0, "limit"), (("streams",), 0, "streams")]:
        with pytest.raises(ConfigError, match=word):
            LafanexConfig.from_dict(broken(path, value))


def test_the_architecture_is_found_by_config_json_and_a_wrong_checkpoint_is_named(tmp_path_factory):
    from roost_b200 import registry
    assert registry.resolve(ConfigReader(LM.MIXED, "config")).name == "Lafanex"
    folder, cfg, _ = model_dir(tmp_path_factory, "mixed", LM.MIXED, seed=5)
    model = H.make_model(folder, torch.float32, "fake")
    # every pass of the looped layers has a cache or state of its own; a layer without a feed-forward loads no second norm
    assert [n.kind for n in model.cache_needs] == ["paged", "state", "paged", "state", "paged", "state"]
    assert sum(1 for g in StepExecutor(model, page_size=4, num_pages=8, max_requests=2).groups for _ in g.runs) == 6
    tensors = LM.draw_tensors(cfg, 5)
    del tensors["l1.mlp.e3.up"]
    tensors["l3.mix.D"] = tensors["l3.mix.D"][:1]
    bad = LM.write_model(tmp_path_factory.mktemp("lafanex_bad"), cfg, tensors)
    with pytest.raises(WeightError) as e:
        H.make_model(bad, torch.float32, "fake")
    assert "l1.mlp.e3.up" in e.value.missing and e.value.wrong_shape[0][0] == "l3.mix.D"


def test_the_random_weights_mode_writes_a_folder_the_engine_runs(tmp_path):
    from roost_b200.weights.random_init import write_random_model
    folder = write_random_model(tmp_path / "m", LM.PLAIN, seed=3, std=0.1, norm_std=0.0)
    model = H.make_model(folder, torch.float32, "fake")
    ex = StepExecutor(model, page_size=4, num_pages=16, max_requests=2)
    out = ex.step([StepEntry("a", [1, 2, 3], [2])])
    assert out.shape == (1, LM.PLAIN["vocab"]) and bool(torch.isfinite(out).all())
