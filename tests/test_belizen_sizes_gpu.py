"""Belizen configurations drawn at random (seeded): every size and constant varies, including the ones the fixed test
models happen to make equal or 1; head sizes of 64 and 128 with equal value heads send bfloat16 runs to the
tensor-core attention kernels, all others to the generic one; windows from one position to more than the prompt with
none to many kept first positions, and no window; rotation of 2 channels to whole heads, interpolated or not, or none;
recurrent heads whose sizes are no multiple of 4 (the scan's copies then move 4 bytes at a time), ranks from 1; experts
with and without pass-through ones and a shared one; loops anywhere, once to three times, and none; any order of
layers.  Each model runs a prompt whole, in portions, its tail token by token and in a batch of two unequal requests,
in float32 (free routing) and bfloat16 (routing pinned by the corrections), against the plain model."""
import random

import pytest
import torch

import belizen_models as bm
from conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 5e-2}        # observed over the fourteen: 2e-5 and 2.4e-2


def draw_config(seed: int) -> dict:
    rng = random.Random(9000 + seed)
    width = rng.choice([40, 64, 72, 96, 100, 128, 136])

    def mlp():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.45:
            return bm.dense(rng.choice([8, 20, 24, 40, 72, 130]))
        experts = rng.choice([1, 2, 3, 5, 8, 12])
        identity = rng.choice([None, 0, 1, 3, 7])
        top = rng.randint(1, min(6, experts + (identity or 0)))
        shared = None if rng.random() < 0.4 else (rng.choice([8, 24, 40, 100]), rng.choice([0.5, 1.5, 7.0]))
        return bm.moe(experts=experts, top=top, ff=rng.choice([8, 16, 24, 40, 64]), limit=rng.choice([0.5, 1.0, 3.0]),
                      identity=identity, shared=shared)

    def attention_layer():
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([8, 16, 24, 40, 64, 64, 128])
        vdim = dim if dim in (64, 128) and rng.random() < 0.7 else rng.choice([8, 12, 16, 40, 64])
        size = rng.choice([None, 1, 5, 33, 64, 65, 90, 128, 1000])
        keep = None if size is None else rng.choice([None, 0, 1, 7, 64, 70, 130])
        rot = rng.choice([None] + [r for r in (2, 4, 8, 16, 32, 64, 128) if r <= dim] + [dim])
        scaling = None
        if rot is not None and rng.random() < 0.6:
            scaling = (rng.choice([1.5, 4.0, 16.0]), rng.choice([32, 256, 4096]), rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))
        return bm.layer("attention", bm.attn(heads=kv * rng.choice([1, 2, 4, 5]), kv=kv, dim=dim, vdim=vdim, scale=rng.uniform(0.05, 0.4),
                                             cap=rng.choice([None, 3.0, 15.0, 50.0]), size=size, keep=keep,
                                             base=rng.choice([100.0, 1e4, 5e5]), rot=rot, scaling=scaling), mlp())

    def gla_layer():
        return bm.layer("gla", bm.gla(heads=rng.choice([1, 2, 3, 4]), dim=rng.choice([4, 9, 16, 40, 64, 130]),
                                      vdim=rng.choice([6, 8, 17, 32, 64, 100]), tau=rng.choice([1.0, 4.0, 16.0, 50.0]),
                                      rank=rng.choice([1, 3, 8, 16, 21])), mlp())

    n = rng.choice([1, 2, 3, 4, 5])
    layers = [attention_layer() if rng.random() < 0.55 else gla_layer() for _ in range(n)]
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(n)
        loop = (start, rng.randint(start + 1, n), rng.choice([1, 2, 3]))
    return bm.model(vocab=rng.choice([97, 160, 301]), width=width, eps=rng.choice([1e-5, 1e-6]), scale=rng.choice([1.0, 5.0, 11.3]),
                    mult=rng.choice([1.0, 0.75, 0.35]), cap=rng.choice([None, 25.0, 60.0]), layers=layers, loop=loop)


@pytest.mark.parametrize("seed", list(range(14)))
def test_random_configuration(seed, tmp_path):
    from rust_inference_b200.engine.engine import Engine
    cfg = draw_config(seed)
    vocab = cfg["vocab"]
    a, b = random_tokens(150, vocab, seed), random_tokens(37, vocab, seed + 100)
    for dtype in ("float32", "bfloat16"):
        model = bm.make(tmp_path, f"r{seed}{dtype}", seed=seed, cfg=cfg, pin_routing=dtype == "bfloat16", drop_rank=seed % 2 == 1)
        want_a, want_b = model.plain_logits(a), model.plain_logits(b)
        eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=1024, n_slots=4)
        s = eng.alloc_slot()
        assert rel_err(eng.step([s], [a], "all"), want_a) < TOL[dtype], (seed, dtype, "whole", cfg)
        eng.free_slot(s)
        s = eng.alloc_slot()                    # the freed slot again, in portions down to two tokens
        rows, at = [], 0
        for take in (66, 2, 63, 2, 17):
            rows.append(eng.step([s], [a[at:at + take]], "all").cpu())
            at += take
        assert rel_err(torch.cat(rows), want_a) < TOL[dtype], (seed, dtype, "portions", cfg)
        eng.free_slot(s)
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([sa, sb], [a[:131], b[:30]], "all").cpu()
        rows_a, rows_b = [out[:131]], [out[131:]]
        for p in range(7):
            out = eng.step([sa, sb], [[a[131 + p]], [b[30 + p]]], "last").cpu()
            rows_a.append(out[0:1])
            rows_b.append(out[1:2])
        eng.free_slot(sb)
        for p in range(138, 150):
            rows_a.append(eng.step([sa], [[a[p]]], "last").cpu())
        assert rel_err(torch.cat(rows_a), want_a) < TOL[dtype], (seed, dtype, "batch a", cfg)
        assert rel_err(torch.cat(rows_b), want_b) < TOL[dtype], (seed, dtype, "batch b", cfg)
        eng.check_device_status()
