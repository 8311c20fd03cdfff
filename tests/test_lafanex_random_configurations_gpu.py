"""Lafanex models drawn at random (layer order, every size, streams or none, a looped range, routing with and without identity
experts and a shared expert, constants), each run through the step function in random portions and batches with pages and slots
used again, against the plain implementation. float32 holds every draw to tight bounds: faults of indexing (a page, a slot, a
tile's or a chunk's edge, a head's group) show there. In bfloat16 the runs follow the engine's routing and are held to the median
over a request's positions of the per-position error: what they add is that every drawn size finds a bfloat16 kernel that serves
it (keys and values of one size on the tensor-core kernels, every other on the 32-bit kernel; every form of the experts'
products), with the strides and alignments it brings."""
import random

import pytest
import torch

from tests import helpers as H
from tests import lafanex_models as LM
from tests.plain import lafanex_plain as P
from tests.test_lafanex import Run

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72, 96, 136, 200])
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 2, 3, 4])
            dim = rng.choice([4, 6, 8, 16, 24, 32, 64])
            vdim = dim if rng.random() < 0.4 else rng.choice([3, 8, 16, 40, 80])
            rot = rng.choice([r for r in (2, 4, 8, 16, 32, 64) if r <= dim])
            layer = LM.attention(heads=kv_heads * rng.choice([1, 2, 3, 4, 10]), kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot,
                                 base=rng.choice([50.0, 10000.0, 1000000.0]), scale=rng.choice([0.05, 0.125, 0.3]) * (16.0 / dim) ** 0.5)
        else:
            layer = LM.mamba(inner=rng.choice([6, 16, 40, 72, 130]), state=rng.choice([1, 4, 8, 16, 24, 48, 70]), dt_rank=rng.choice([1, 2, 5, 8, 16]),
                             conv=rng.randint(1, 5))
        kind = rng.random()
        if kind < 0.15:
            mlp = None
        elif kind < 0.45:
            mlp = LM.dense(ff=rng.choice([16, 48, 128]))
        else:
            experts = rng.randint(1, 12)
            identity = rng.choice([0, 0, 1, 3])
            mlp = LM.moe(experts=experts, identity=identity, top=rng.randint(1, min(4, experts + identity)), ff=rng.choice([8, 64, 128]),
                         limit=rng.choice([0.5, 2.0, 7.0]), scale=rng.choice([1.0, 2.5]), shared=rng.choice([0, 32, 128]), shared_limit=rng.choice([1.0, 5.0]))
        layers.append((layer, mlp))
    loop = None
    if rng.random() < 0.6:
        a = rng.randrange(len(layers))
        loop = (a, rng.randint(a + 1, len(layers)), rng.randint(1, 3))
    return LM.config(layers, width=width, vocab=rng.randint(50, 500), eps=rng.choice([1e-5, 1e-6]), streams=rng.choice([None, 1, 2, 4, 5]), loop=loop)


def run_draw(tmp_path, seed: int, dtype) -> None:
    cfg = draw_config(seed)
    rng = random.Random(seed * 7 + 1)
    tensors = LM.draw_tensors(cfg, seed)
    folder = LM.write_model(tmp_path, cfg, tensors)
    weights = LM.plain_weights(tensors)
    page = rng.choice([4, 8, 16])
    run = Run(folder, cfg, ("gpu", dtype), page_size=page, num_pages=3 * (-(-330 // page)) + 2, slots=3)
    reqs = {f"q{i}": H.random_ids(rng.choice([1, 2, 7, 40, 131, 300]), cfg["vocab"], seed * 13 + i) for i in range(5)}
    waiting, live = list(reqs), {}
    while waiting or live:
        while waiting and len(live) < 3:
            live[waiting.pop(0)] = 0
        entries = []
        for rid in [r for r in live if rng.random() < 0.8] or [next(iter(live))]:
            left = len(reqs[rid]) - live[rid]
            n = 1 if left <= 5 else min(left - 5, rng.choice([2, 3, 9, 33, 64, 200]))
            entries.append((rid, reqs[rid][live[rid] : live[rid] + n]))
            live[rid] += n
        run.step(entries)
        for rid, _ in entries:
            if live[rid] == len(reqs[rid]):
                run.finish(rid)
                del live[rid]
    for rid, ids in reqs.items():
        if dtype == torch.float32:
            run.check(rid, ids, weights, f"draw {seed} {rid}", f32_bounds=(2e-3, 5e-5))
            continue
        got = torch.cat(run.logits.pop(rid)).double()
        forced = {r: torch.cat(v) for r, v in run.forced.pop(rid, {}).items()}
        want = P.forward(cfg, weights, list(ids), forced=forced, slack=float("inf"))
        per_position = ((got - want) ** 2).mean(1).sqrt() / (want ** 2).mean().sqrt()
        assert torch.isfinite(got).all() and float(per_position.median()) < 0.08, (seed, rid, float(per_position.median()))
    assert run.all_free()
    run.model.rt.kernels.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34, 55, 89])
def test_random_configurations_in_random_portions_and_batches(tmp_path, seed, dtype):
    run_draw(tmp_path, seed, dtype)
