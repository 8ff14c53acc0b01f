"""Small Belizen configurations for the tests, random weights for them, and model folders made from both.

The configurations differ from one another in every size and constant and include values that make two sizes equal or
1: one kv head per query head and one for all, a single head, windows of one position, of less than a page and of more
than two pages, kept first positions fewer and more than the window and none, rotation of a whole head and of two
channels, with and without interpolated frequencies, no rotation, no cap, value heads narrower and wider than key
heads, decays of rank 1 and of ranks that are no multiple of 4, one expert chosen, experts that hand their input
through in the majority and none at all, no shared expert, layers without feed-forward, a run of layers passed once,
twice and three times, starting at the first layer and ending at the last, no loop, widths that are no multiple of 32."""
import json
import os

import torch

import plain_belizen


def attn(*, heads, kv, dim, vdim, scale, cap=None, size=None, keep=None, base=None, rot=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if cap is not None:
        m["softcap"] = cap
    if size is not None:
        m["mask"] = {"size": size}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def gla(*, heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(*, experts, top, ff, limit, identity=None, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if identity is not None:
        out["router"]["identity"] = identity
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(*, vocab, width, eps, scale, mult, layers, cap=None, loop=None):
    out = {"architecture": "Belizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "residual_mult": mult, "layers": layers}
    if cap is not None:
        out["logit_softcap"] = cap
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


CONFIGS = {
    # a window inside a page with three kept positions, a window across pages with more kept than half of it; the
    # middle two layers passed three times; more pass-through experts than real ones
    "A": model(vocab=211, width=96, eps=1e-5, scale=3.0, mult=0.6, cap=12.0, loop=(1, 3, 3), layers=[
        layer("attention", attn(heads=4, kv=2, dim=16, vdim=24, scale=0.2, cap=30.0, size=20, keep=3, base=5000.0, rot=8,
                                scaling=(3.0, 64, 8.0, 0.5)), dense(72)),
        layer("gla", gla(heads=3, dim=24, vdim=40, tau=8.0, rank=5),
              moe(experts=3, top=3, ff=24, limit=0.8, identity=5, shared=(40, 1.2))),
        layer("attention", attn(heads=2, kv=2, dim=8, vdim=8, scale=0.4, cap=12.0, size=150, keep=70, base=100.0, rot=8), None),
        layer("gla", gla(heads=1, dim=72, vdim=33, tau=1.0, rank=1), moe(experts=5, top=1, ff=16, limit=2.0)),
    ]),
    # width 72; single heads; a window of one position with one kept; no cap on scores or logits; no rotation in one
    # layer and two channels in another; the whole model is the loop, passed twice; no pass-through experts
    "B": model(vocab=157, width=72, eps=1e-6, scale=1.0, mult=1.0, loop=(0, 3, 2), layers=[
        layer("gla", gla(heads=2, dim=8, vdim=16, tau=20.0, rank=12), dense(40)),
        layer("attention", attn(heads=1, kv=1, dim=24, vdim=24, scale=0.2, size=1, keep=1), moe(experts=6, top=2, ff=20, limit=1.0,
                                                                                               identity=0, shared=(12, 0.7))),
        layer("attention", attn(heads=3, kv=1, dim=8, vdim=16, scale=0.3, cap=15.0, size=33, keep=0, base=1e6, rot=2), dense(56)),
    ]),
    # sizes the tensor-core kernels take (heads of 64 and 128, widths that are multiples of 8), windows across
    # pages; no loop; causal attention without a window
    "C": model(vocab=264, width=256, eps=1e-6, scale=16.0, mult=0.8, cap=20.0, layers=[
        layer("attention", attn(heads=4, kv=2, dim=64, vdim=64, scale=0.125, cap=30.0, size=70, keep=10, base=500000.0, rot=32,
                                scaling=(8.0, 256, 16.0, 2.0)), dense(384)),
        layer("gla", gla(heads=4, dim=64, vdim=64, tau=10.0, rank=24),
              moe(experts=6, top=3, ff=48, limit=1.25, identity=3, shared=(96, 2.0))),
        layer("attention", attn(heads=2, kv=1, dim=128, vdim=128, scale=0.09, cap=20.0, size=129, keep=64, base=10000.0, rot=128),
              moe(experts=4, top=2, ff=128, limit=1.5, identity=1)),
        layer("attention", attn(heads=8, kv=2, dim=64, vdim=64, scale=0.1, cap=25.0, base=10000.0, rot=64), dense(128)),
    ]),
}


def random_weights(cfg, seed, pin_routing=True, hot=1.0):
    """Random tensors for a configuration, every value a bfloat16 number: matrices ~ N(0, 1/sqrt(inputs)), norm
    weights 1 + N(0, 0.2), biases and the vectors that join the stream at a pass of their own scale.  With
    pin_routing the corrections are 1.5 apart, so they decide the choice by themselves (a softmax score lies in
    (0, 1)) and a bfloat16 run chooses the experts the plain model chooses; the weights still come from the router."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in plain_belizen.tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / max(cfg["embedding"]["scale"], 1.0)
        elif name == "loop.step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("a2.b"):
            t = 1.0 + torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "correction":
            if pin_routing:
                t = 1.5 * torch.randperm(shape[0], generator=g).float() - 4.0
            else:
                t = 0.05 * torch.randn(shape, generator=g)
        elif leaf == "router":
            t = hot * 2.0 * torch.randn(shape, generator=g) / shape[-1] ** 0.5
        elif leaf == "a2":
            t = 2.0 * torch.randn(shape, generator=g) / shape[-1] ** 0.5
        else:
            t = hot * torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


class BelizenModel:
    def __init__(self, folder, cfg, weights):
        self.folder, self.cfg = folder, cfg
        self.weights = {k: v.float() for k, v in weights.items()}       # the stored bfloat16 values, widened

    def plain_logits(self, tokens, **kw):
        return plain_belizen.forward(self.cfg, self.weights, tokens, **kw)


def make(tmp_path, name, seed=0, cfg=None, edit=None, pin_routing=True, drop_rank=False):
    """A model folder.  drop_rank: config.json leaves the decays' rank to the shape of the tensor that has it."""
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    weights = random_weights(cfg, seed, pin_routing=pin_routing)
    if edit is not None:
        edit(weights)
    folder = str(tmp_path / f"belizen_{name}_{seed}")
    os.makedirs(folder, exist_ok=True)
    stored = cfg
    if drop_rank:
        stored = dict(cfg, layers=[dict(L, mixer={k: v for k, v in L["mixer"].items() if k != "rank"}) if L["type"] == "gla" else L
                                   for L in cfg["layers"]])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(stored, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return BelizenModel(folder, cfg, weights)
