"""The Vamatar decoder through the engine's step function, cache manager, scheduler and entry point, against the plain
implementation of tests/plain/vamatar_plain.py, for every way of cutting the work.

Each test runs on the GPU with the real kernel library in float32 (captured steps) and bfloat16 (marked gpu), and on the
CPU with the stand-in kernels of tests/fake_kernels.py, which checks the host side. In bfloat16 the engine's routing
choices are recorded and handed to the plain implementation, which checks that each was within a rounding of the best
(two nearly equal scores may be ordered differently in lower precision); float32 runs choose for themselves.
"""
import random

import pytest
import torch

from roost_b200 import GenerationOptions, RoostEngine
from roost_b200.config.reader import ConfigError, ConfigReader
from roost_b200.config.vamatar import VamatarConfig
from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.loader import WeightError
from tests import helpers as H
from tests import vamatar_models as VM
from tests.plain import vamatar_plain as P

BACKENDS = [
    pytest.param(("gpu", torch.float32), id="gpu-f32", marks=pytest.mark.gpu),
    pytest.param(("gpu", torch.bfloat16), id="gpu-bf16", marks=pytest.mark.gpu),
    pytest.param(("fake", torch.float32), id="cpu-fake"),
]
F32_WORST, F32_RMS = 1e-4, 1e-5
BF16_WORST, BF16_RMS = 0.5, 0.04     # the worst of tens of thousands of logits is the tail of the rounding noise; the root mean square is what a fault moves
ROUTE_SLACK = 0.25            # in router logits: what bfloat16 inputs may move a logit of size ten by


@pytest.fixture(params=BACKENDS)
def backend(request):
    return request.param


_MODELS: dict = {}


def model_dir(tmp_path_factory, name, cfg, seed, change=None):
    """A model folder written once a session; ``change(cfg, tensors)`` edits the drawn weights first."""
    if name not in _MODELS:
        tensors = VM.draw_tensors(cfg, seed)
        if change is not None:
            change(cfg, tensors)
        _MODELS[name] = (VM.write_model(tmp_path_factory.mktemp(f"vamatar_{name}"), cfg, tensors), cfg, VM.plain_weights(tensors))
    return _MODELS[name]


class Run:
    """Drives a StepExecutor and keeps, per request, the logits of every position and (when recording) the experts the
    engine chose in every routed layer."""

    def __init__(self, model_dir, cfg, backend, page_size=4, num_pages=64, slots=4):
        kind, self.dtype = backend
        self.cfg = cfg
        self.model = H.make_model(model_dir, self.dtype, kind)
        # bfloat16 steps run uncaptured so that the routing recorder sees every call; float32 steps replay graphs
        self.record = self.dtype == torch.bfloat16
        self.ex = StepExecutor(self.model, page_size=page_size, num_pages=num_pages, max_requests=slots, use_graphs=not self.record)
        self.routed = VM.routed_layers(cfg)
        self.logits: dict = {}
        self.forced: dict = {}

    def step(self, entries):
        """entries: [(request id, tokens)]; every position's logits are asked for."""
        step_entries = [StepEntry(rid, list(toks), list(range(len(toks)))) for rid, toks in entries]
        if self.record:
            with VM.RouteRecorder(self.model.rt.kernels) as rec:
                out = self.ex.step(step_entries)
            assert len(rec.calls) == len(self.routed)
        else:
            out = self.ex.step(step_entries)
        at = 0
        for rid, toks in entries:
            n = len(toks)
            self.logits.setdefault(rid, []).append(out[at : at + n].float().cpu())
            if self.record:
                for layer, call in zip(self.routed, rec.calls):
                    self.forced.setdefault(rid, {}).setdefault(layer, []).append(call[at : at + n])
            at += n
        self.ex.cache.check_invariants()

    def finish(self, rid):
        self.ex.finish(rid)

    def check(self, rid, ids, weights, what, bf16_bounds=(BF16_WORST, BF16_RMS), slack=ROUTE_SLACK, f32_bounds=(F32_WORST, F32_RMS)):
        got = torch.cat(self.logits.pop(rid))
        forced = {layer: torch.cat(v) for layer, v in self.forced.pop(rid, {}).items()} if self.record else None
        n = got.shape[0]
        want = P.forward(self.cfg, weights, list(ids[:n]), forced=forced, slack=slack)
        err, rms = H.scaled_error(got, want), H.rms_error(got, want)
        print(f"MEASURED {what} {self.dtype}: worst scaled error {err:.3e}, rms error {rms:.3e}")
        worst, bound = f32_bounds if self.dtype == torch.float32 else bf16_bounds
        assert err < worst and rms < bound, f"{what}: worst scaled error {err}, rms error {rms}"
        return got, want

    def all_free(self):
        return all(p.used_count == 0 for p in self.ex.cache.pools)


def ids_for(cfg, n, seed):
    return H.random_ids(n, cfg["vocab"], seed)


SINGLE = {
    "latent_only": VM.config([(VM.latent(heads=2, dim=6, rot_dim=6, vdim=5, kv_rank=7, window=5, dims=6), None)], width=24, vocab=50),
    "mamba_only": VM.config([(VM.mamba(heads=3, vdim=5, state=6, groups=1, conv=4, norm_groups=3), None)], width=20, vocab=45, cap=None),
    "dense_after_latent": VM.config([(VM.latent(window=None), VM.dense(ff=17))], width=28, vocab=33),
    "experts_after_mamba": VM.config([(VM.mamba(), VM.moe(experts=6, top=2, ff=9, shared=11))], width=32, vocab=40),
}
ALL = dict(VM.CONFIGS, **SINGLE)


@pytest.fixture(params=sorted(ALL))
def any_model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, ALL[request.param], seed=len(request.param))


@pytest.fixture(params=sorted(VM.CONFIGS))
def model(request, tmp_path_factory):
    return (request.param,) + model_dir(tmp_path_factory, request.param, VM.CONFIGS[request.param], seed=len(request.param))


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("length", [1, 2, 3, 37, 150])
def test_each_mechanism_and_each_model_on_whole_prompts(any_model, backend, length):
    """Models of one mechanism each (latent attention alone, the recurrence alone, each feed-forward) and the mixed models;
    the shortest prompts are the first tokens of a sequence: the convolution's zeros before the start, an empty state, a
    window that holds less than its size."""
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


def test_long_decoding_past_every_window_and_many_pages(model, backend):
    name, folder, cfg, weights = model
    run = Run(folder, cfg, backend, page_size=4, num_pages=80)
    ids = ids_for(cfg, 230, seed=3)
    run.step([("r", ids[:3])])
    for t in ids[3:]:
        run.step([("r", [t])])
    windowed = [g for g in run.ex.groups if g.kind == "paged" and g.window is not None]
    for g in windowed:      # the pages a window has passed went back to the pool
        gi = run.ex.groups.index(g)
        assert run.ex.cache.held("r")[gi] <= -(-g.window // 4) + 1
    run.finish("r")
    run.check("r", ids, weights, f"{name} long decoding")


LONG = VM.config([(VM.latent(heads=4, dim=16, rot_dim=8, vdim=8, kv_rank=32, window=80, base=10000.0), VM.moe(experts=5, top=2, ff=128, shared=40)),
                  (VM.mamba(heads=2, vdim=16, state=16, groups=1, conv=4, norm_groups=1), VM.moe(experts=3, top=2, ff=256, shared=0))],
                 width=72, vocab=83)


def test_a_long_prompt_takes_the_forms_of_steps_of_many_rows(tmp_path_factory, backend):
    """600 tokens in one step and then 2 + 1: on the device in bfloat16 the experts' products run on the grouped tcgen05
    kernel (1,200 sorted rows, an expert size that is a multiple of 128, a width of 72 that is no multiple of its 64-wide
    k blocks), the attention on the tensor cores and the recurrence in chunks; the other backends take their own forms of
    the same step."""
    folder, cfg, weights = model_dir(tmp_path_factory, "long", LONG, seed=21)
    run = Run(folder, cfg, backend, page_size=16, num_pages=48)
    ids = ids_for(cfg, 603, seed=8)
    run.step([("r", ids[:600])])
    run.step([("r", ids[600:602])])
    run.step([("r", ids[602:])])
    run.finish("r")
    run.check("r", ids, weights, "long prompt")


# ------------------------------------------------------------------------------------------------ keys that must (not) be seen
WINDOW = 9
EDGE = VM.config([(VM.latent(heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=10, window=WINDOW), VM.dense(ff=20)),
                  (VM.latent(heads=3, dim=5, rot_dim=4, vdim=4, kv_rank=10, window=WINDOW + 4, kv_from=0), None)], width=32, vocab=53)
FAR = VM.config([(VM.latent(heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=10, window=None), None), (VM.mamba(), VM.dense(ff=16))],
                width=32, vocab=53)
KEY, QUERY = 7, 11        # token ids: QUERY scores KEY far above every other key in the first layer


def sharpened(tmp_path_factory, name, cfg):
    return model_dir(tmp_path_factory, name, cfg, seed=77, change=lambda c, t: VM.sharpen(c, t, KEY, QUERY))


def filler(cfg, n, seed):
    rng = random.Random(seed)
    return [rng.choice([t for t in range(cfg["vocab"]) if t not in (KEY, QUERY)]) for _ in range(n)]


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
def test_a_key_just_inside_and_just_outside_the_window_at_every_page_offset(tmp_path_factory, backend, decoded):
    """The key token sits ``distance`` places before the query token; with distance = window - 1 it is the oldest key the
    window keeps, with distance = window the first one it has dropped. The sharpened weights put nearly all of the query's
    attention on that key when it is seen, so a window that is one off changes the query's logits by far more than the
    bound. The key's place runs through every offset of a page of four."""
    folder, cfg, weights = sharpened(tmp_path_factory, "edge", EDGE)
    run = Run(folder, cfg, backend, page_size=4, num_pages=40)
    seen_outputs = {}
    for distance in (WINDOW - 1, WINDOW):
        for at in (13, 14, 15, 16, 17):
            ids = filler(cfg, 34, seed=at)
            ids[at], ids[at + distance] = KEY, QUERY
            rid = f"d{distance}a{at}"
            if decoded:
                run.step([(rid, ids[: at + 1])])
                for t in ids[at + 1 :]:
                    run.step([(rid, [t])])
            else:
                run.step([(rid, ids[:5])])
                run.step([(rid, ids[5:])])
            run.finish(rid)
            got, want = run.check(rid, ids, weights, f"edge distance {distance} key at {at}")
            seen_outputs[(distance, at)] = want[at + distance]
    # the test's own sharpness: seeing the key or not moves the plain logits of the query's position by much more than the bound
    for at in (13, 14, 15, 16, 17):
        moved = H.rms_error(seen_outputs[(WINDOW - 1, at)][None], seen_outputs[(WINDOW, at)][None])
        assert moved > 0.1, moved


@pytest.mark.parametrize("decoded", [False, True], ids=["in a prompt", "decoded"])
def test_a_key_far_away_among_hundreds(tmp_path_factory, backend, decoded):
    folder, cfg, weights = sharpened(tmp_path_factory, "far", FAR)
    run = Run(folder, cfg, backend, page_size=4, num_pages=120)
    outputs = []
    for key_there in (True, False):
        ids = filler(cfg, 330, seed=4)
        if key_there:
            ids[2] = KEY
        ids[321] = QUERY
        rid = f"far{key_there}"
        if decoded:
            run.step([(rid, ids[:300])])
            for t in ids[300:]:
                run.step([(rid, [t])])
        else:
            run.step([(rid, ids[:130])])
            run.step([(rid, ids[130:])])
        run.finish(rid)
        got, want = run.check(rid, ids, weights, f"far key present {key_there}")
        outputs.append(want[321])
    assert H.rms_error(outputs[0][None], outputs[1][None]) > 0.1


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
    cfg = VamatarConfig.from_dict(VM.MIXED)
    spec = cfg.to_spec()
    assert spec.architecture == "Vamatar" and len(spec.blocks) == 4
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, 0, None]
    # the shared latent cache is kept for the wider of the two windows; each layer masks by its own
    assert spec.blocks[0].mixer.window == 9 and spec.blocks[2].mixer.window == 14
    assert spec.blocks[0].mixer.cache_window == spec.blocks[2].mixer.cache_window == 14
    assert spec.blocks[3].feed_forward is None and spec.blocks[3].post_mixer_norm is None
    assert spec.embedding.scale == 0.7 and spec.head.cap == 9.0
    odd = VamatarConfig.from_dict(VM.ODD).to_spec()
    assert odd.head.kind == "linear" and odd.blocks[1].mixer.cache_window is None and odd.blocks[2].mixer.window == 6
    assert odd.blocks[1].mixer.position.rotary_dim == 4 and odd.blocks[1].mixer.rope_dim == 8

    def broken(path, value):
        import copy
        c = copy.deepcopy(VM.MIXED)
        node = c
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        return c

    for path, value, word in [(("layers", 2, "mixer", "kv_from"), 1, "kv_from"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
                              (("layers", 2, "mixer", "kv_rank"), 11, "kv_rank"), (("layers", 1, "type"), "lstm", "type"),
                              (("layers", 1, "mlp", "kind"), "sparse", "kind"), (("layers", 1, "mlp", "router", "top"), 9, "top"),
                              (("layers", 1, "mixer", "groups"), 3, "groups"), (("norm",), None, "norm.eps"), (("width",), 0, "width"),
                              (("layers", 0, "mixer", "rot", "dims"), 3, "dims")]:
        with pytest.raises(ConfigError, match=word):
            VamatarConfig.from_dict(broken(path, value))


def test_the_architecture_is_found_by_config_json_and_a_wrong_checkpoint_is_named(tmp_path_factory):
    from roost_b200 import registry
    from roost_b200.weights.safetensors_io import write_safetensors
    assert registry.resolve(ConfigReader(VM.MIXED, "config")).name == "Vamatar"
    folder, cfg, _ = model_dir(tmp_path_factory, "mixed", VM.MIXED, seed=5)
    model = H.make_model(folder, torch.float32, "fake")
    assert [n.kind if n else None for n in model.cache_needs] == ["paged", "state", None, "state"]
    tensors = VM.draw_tensors(cfg, 5)
    del tensors["l1.mlp.e3.up"]
    tensors["l3.mix.D"] = tensors["l3.mix.D"][:1]
    bad = VM.write_model(tmp_path_factory.mktemp("vamatar_bad"), cfg, tensors)
    with pytest.raises(WeightError) as e:
        H.make_model(bad, torch.float32, "fake")
    assert "l1.mlp.e3.up" in e.value.missing and e.value.wrong_shape[0][0] == "l3.mix.D"
