"""Small Redodra configurations for the tests, and model folders made from them.

They differ from one another in every size and constant and include values that make two sizes equal or 1: one kv
head per query head and one for all, a single head, windows of one position, of less than a page and of more than two
pages, kept first positions fewer and more than the window, none kept, rotation of a whole head and of a few channels,
convolutions of one to five taps, a state of one row, one and several groups, norm groups equal to and different from
the heads, value heads narrower and wider than key heads, layers that read an earlier layer's keys (also two of them,
also as the last layer), layers without feed-forward, widths that are no multiple of 32."""
import json
import os

import plain_redodra


def attn(*, heads, kv, dim, vdim, scale, cap, base, rot, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap,
         "rot": {"base": base, "dims": rot}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def window(*, heads, kv, dim, vdim, scale, cap, size, keep):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap,
            "mask": {"size": size, "keep_first": keep}}


def ssm(*, heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def delta(*, heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def side(left, right):
    return {"left": left, "right": right}


CONFIGS = {
    # a window inside a page with three kept positions, one across pages with more kept than half of it; two readers
    # of layer 1's keys, the last of them the last layer
    "A": {"architecture": "Redodra", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "layers": [
        layer("parallel", side(window(heads=4, kv=2, dim=16, vdim=24, scale=0.2, cap=30.0, size=20, keep=3),
                               ssm(heads=3, vdim=16, state=8, groups=1, conv=4, norm_groups=1)), 72),
        layer("attention", attn(heads=4, kv=1, dim=32, vdim=16, scale=0.15, cap=20.0, base=5000.0, rot=8), 80),
        layer("delta", delta(heads=4, kv=2, dim=16, vdim=24, conv=3), None),
        layer("attention", attn(heads=2, kv=1, dim=32, vdim=16, scale=0.3, cap=8.0, base=5000.0, rot=8, kv_from=1), 40),
        layer("parallel", side(window(heads=2, kv=2, dim=8, vdim=8, scale=0.4, cap=12.0, size=150, keep=70),
                               ssm(heads=4, vdim=8, state=24, groups=2, conv=2, norm_groups=4)), None),
        layer("attention", attn(heads=3, kv=1, dim=32, vdim=16, scale=0.2, cap=50.0, base=5000.0, rot=8, kv_from=1), 56),
    ]},
    # width 72; single heads; a window of one position with one kept; convolutions of one tap; a state of one row
    "B": {"architecture": "Redodra", "vocab": 157, "width": 72, "norm": {"eps": 1e-6}, "layers": [
        layer("delta", delta(heads=1, kv=1, dim=40, vdim=72, conv=1), 40),
        layer("parallel", side(window(heads=1, kv=1, dim=24, vdim=24, scale=0.2, cap=5.0, size=1, keep=1),
                               ssm(heads=1, vdim=40, state=1, groups=1, conv=1, norm_groups=1)), 24),
        layer("attention", attn(heads=3, kv=3, dim=8, vdim=8, scale=0.35, cap=1000.0, base=1e6, rot=8), 56),
        layer("delta", delta(heads=6, kv=2, dim=8, vdim=8, conv=5), None),
        layer("parallel", side(window(heads=3, kv=1, dim=8, vdim=16, scale=0.3, cap=15.0, size=33, keep=0),
                               ssm(heads=2, vdim=12, state=20, groups=2, conv=3, norm_groups=3)), 40),
    ]},
    # sizes the tensor-core kernels take: heads of 64 and 128, windows across pages
    "C": {"architecture": "Redodra", "vocab": 264, "width": 256, "norm": {"eps": 1e-6}, "layers": [
        layer("attention", attn(heads=4, kv=2, dim=64, vdim=64, scale=0.125, cap=30.0, base=500000.0, rot=32), 384),
        layer("parallel", side(window(heads=4, kv=2, dim=64, vdim=64, scale=0.125, cap=40.0, size=70, keep=10),
                               ssm(heads=8, vdim=32, state=64, groups=2, conv=4, norm_groups=2)), 256),
        layer("delta", delta(heads=4, kv=4, dim=64, vdim=128, conv=4), 384),
        layer("attention", attn(heads=8, kv=2, dim=64, vdim=64, scale=0.1, cap=25.0, base=500000.0, rot=32, kv_from=0), 128),
        layer("parallel", side(window(heads=2, kv=1, dim=128, vdim=128, scale=0.09, cap=20.0, size=129, keep=64),
                               ssm(heads=2, vdim=64, state=128, groups=1, conv=4, norm_groups=4)), None),
    ]},
}


class RedodraModel:
    def __init__(self, folder, cfg, weights):
        self.folder, self.cfg = folder, cfg
        self.weights = {k: v.float() for k, v in weights.items()}       # the stored bfloat16 values, widened

    def plain_logits(self, tokens, **kw):
        return plain_redodra.forward(self.cfg, self.weights, tokens, **kw)


def make(tmp_path, name, seed=0, cfg=None, edit=None, hot=1.0):
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    weights = plain_redodra.random_weights(cfg, seed, hot=hot)
    if edit is not None:
        edit(weights)
    folder = str(tmp_path / f"redodra_{name}_{seed}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return RedodraModel(folder, cfg, weights)
