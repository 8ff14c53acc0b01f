"""Redodra configurations drawn at random (seeded): every size and constant varies, including the ones the fixed
test models happen to make equal or 1; head sizes of 64 and 128 send bfloat16 runs to the tensor-core attention
kernels, all others to the generic one; windows from one position to more than the prompt with none to many kept
first positions; states and value heads that are no multiple of 4 (the scan's copies then move 4 bytes at a time);
any order of layers, readers of an earlier layer's keys anywhere after it.  Each model runs a prompt whole, in
portions, its tail token by token and in a batch of two unequal requests, in float32 and bfloat16, against the plain
model."""
import random

import pytest
import torch

import redodra_models as rm
from conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def draw_config(seed: int) -> dict:
    rng = random.Random(7000 + seed)
    width = rng.choice([40, 64, 72, 96, 100, 128, 136])

    def ff():
        return None if rng.random() < 0.2 else rng.choice([8, 20, 24, 40, 72, 130])

    def head_sizes():
        dim = rng.choice([8, 16, 24, 40, 64, 64, 128])
        return dim, (dim if dim in (64, 128) and rng.random() < 0.7 else rng.choice([8, 12, 16, 40, 64]))

    owners = {}

    def attention_layer(i):
        if owners and rng.random() < 0.4:
            src = rng.choice(list(owners))
            kv, dim, vdim, base, rot = owners[src]
        else:
            src, kv = None, rng.choice([1, 2, 3])
            dim, vdim = head_sizes()
            base = rng.choice([100.0, 1e4, 5e5])
            rot = rng.choice([r for r in (2, 4, 8, 16, 32, 64, 128) if r <= dim] + [dim])
            owners[i] = (kv, dim, vdim, base, rot)
        return rm.layer("attention", rm.attn(heads=kv * rng.choice([1, 2, 4, 5]), kv=kv, dim=dim, vdim=vdim,
                                             scale=rng.uniform(0.05, 0.4), cap=rng.choice([3.0, 15.0, 50.0, 400.0]),
                                             base=base, rot=rot, kv_from=src), ff())

    def delta_layer():
        kv = rng.choice([1, 2, 3])
        return rm.layer("delta", rm.delta(heads=kv * rng.choice([1, 2, 3]), kv=kv, dim=rng.choice([4, 9, 16, 40, 64, 130]),
                                          vdim=rng.choice([6, 8, 17, 32, 64, 100]), conv=rng.choice([1, 2, 3, 4, 5])), ff())

    def parallel_layer():
        kv = rng.choice([1, 2, 3])
        dim, vdim = head_sizes()
        groups = rng.choice([1, 2, 3])
        heads = groups * rng.choice([1, 2, 4])
        vd = rng.choice([6, 8, 12, 32, 64])
        ng = rng.choice([g for g in (1, 2, 3, 4, 6, heads) if (heads * vd) % g == 0])
        size = rng.choice([1, 5, 33, 64, 65, 90, 128, 1000])
        return rm.layer("parallel", rm.side(
            rm.window(heads=kv * rng.choice([1, 2, 4, 6]), kv=kv, dim=dim, vdim=vdim, scale=rng.uniform(0.05, 0.4),
                      cap=rng.choice([3.0, 15.0, 50.0]), size=size, keep=rng.choice([0, 1, 7, 64, 70, 130])),
            rm.ssm(heads=heads, vdim=vd, state=rng.choice([1, 7, 16, 48, 64, 128, 200]), groups=groups,
                   conv=rng.choice([1, 2, 3, 4]), norm_groups=ng)), ff())

    layers = []
    for i in range(rng.choice([2, 3, 4, 5, 6])):
        kind = rng.choice(["attention", "delta", "parallel"])
        layers.append(attention_layer(i) if kind == "attention" else delta_layer() if kind == "delta" else parallel_layer())
    return {"architecture": "Redodra", "vocab": rng.choice([97, 160, 301]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configuration(seed, tmp_path):
    from rust_inference_b200.engine.engine import Engine
    cfg = draw_config(seed)
    vocab = cfg["vocab"]
    a, b = random_tokens(150, vocab, seed), random_tokens(37, vocab, seed + 100)
    model = rm.make(tmp_path, f"r{seed}", seed=seed, cfg=cfg)
    want_a, want_b = model.plain_logits(a), model.plain_logits(b)
    for dtype in ("float32", "bfloat16"):
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
