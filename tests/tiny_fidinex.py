"""Small Fidinex configurations for the tests (and one of whole tiles for long prompts), and model folders with
weights large enough that every mechanism shows in the logits.  They differ from one another in every size and
option: the number of streams (one, several, and none at all: the plain pre-norm layer), the order of the two
mixers, which layer is the first to blend values and which do not blend, layers without feed-forward, query
temperatures with short periods (and none), key/value groups of one, two and all heads, values wider and narrower
than keys, equal widths of 64 and 128 (the tensor-core attention kernels), latent rows wider than 256, widths and
vocabularies that are no multiple of 16."""
import json
import os

import numpy as np


def _att(heads, kv_heads, dim, vdim, scale, q_temp=None, v_mix=False, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if q_temp:
        m["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return dict(type="attention", mixer=m, mlp=mlp)


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp=None):
    return dict(type="latent_attention",
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                           rot=dict(base=base, dims=rot_dim)), mlp=mlp)


def _dense(ff):
    return dict(kind="dense", ff=ff)


FID_A = dict(
    architecture="Fidinex", vocab=301, width=80, norm=dict(eps=1e-5), streams=2,
    layers=[
        _lat(3, 16, 8, 24, 20, 0.2, 100.0, _dense(96)),
        _att(4, 2, 24, 40, 0.3, (0.5, 7), True, _dense(160)),
        _att(2, 2, 32, 32, 0.25, None, False, None),
        _att(6, 2, 16, 40, 0.35, (0.2, 16), True, _dense(64)),
        _att(2, 2, 8, 40, 0.5, (1.0, 3), True, None),
    ])

# one stream that still has its weights; a single attention layer between latent ones
FID_B = dict(
    architecture="Fidinex", vocab=257, width=64, norm=dict(eps=1e-6), streams=1,
    layers=[
        _att(3, 3, 16, 8, 0.3, (0.4, 5), True, _dense(128)),
        _lat(2, 24, 4, 16, 40, 0.15, 7.0, None),
        _lat(5, 8, 16, 12, 12, 0.3, 10000.0, _dense(72)),
    ])

# no streams at all (the plain pre-norm layer); head size 64 with equal value width: the tensor-core attention kernels
FID_C = dict(
    architecture="Fidinex", vocab=512, width=128, norm=dict(eps=1e-5),
    layers=[
        _att(4, 2, 64, 64, 0.125, (0.3, 50), True, _dense(256)),
        _lat(4, 32, 32, 32, 64, 0.12, 1000.0, _dense(192)),
        _att(8, 2, 64, 64, 0.11, None, True, _dense(256)),
    ])

# four streams, a width and a vocabulary that no tensor-core product takes, head size 128, a latent row wider than 256
FID_D = dict(
    architecture="Fidinex", vocab=211, width=100, norm=dict(eps=1e-5), streams=4,
    layers=[
        _att(2, 1, 128, 128, 0.09, (0.3, 20), False, _dense(72)),
        _lat(2, 40, 64, 20, 200, 0.1, 500.0, _dense(40)),
        _att(3, 1, 20, 84, 0.2, None, True, None),
        _att(1, 1, 48, 84, 0.15, (0.7, 11), True, _dense(56)),
    ])

# widths of whole tiles, for prompts of hundreds of tokens: products on tcgen05, attention of head size 64 on the
# tensor-core kernels, three streams
FID_E = dict(
    architecture="Fidinex", vocab=1000, width=256, norm=dict(eps=1e-6), streams=3,
    layers=[
        _lat(4, 64, 32, 64, 128, 0.1, 10000.0, _dense(512)),
        _att(4, 2, 64, 64, 0.125, (0.3, 100), True, _dense(512)),
        _att(4, 1, 64, 64, 0.125, (0.1, 64), False, _dense(256)),
        _att(8, 2, 32, 64, 0.17, None, True, _dense(512)),
    ])

# latent layers whose heads are 64 and 128 wide with values as wide: their prompt portions run on expanded keys and
# values (the tensor-core kernels for prompts), their single tokens in the latent form; two streams
FID_F = dict(
    architecture="Fidinex", vocab=640, width=128, norm=dict(eps=1e-5), streams=2,
    layers=[
        _lat(4, 32, 32, 64, 64, 0.12, 10000.0, _dense(256)),
        _att(2, 2, 64, 64, 0.125, (0.2, 32), True, _dense(128)),
        _lat(2, 64, 64, 128, 256, 0.09, 300.0, _dense(256)),
        _lat(3, 96, 32, 128, 136, 0.1, 50.0, None),
    ])

CONFIGS = {"fid_a": (FID_A, 31), "fid_b": (FID_B, 32), "fid_c": (FID_C, 33), "fid_d": (FID_D, 34), "fid_e": (FID_E, 35), "fid_f": (FID_F, 36)}


def make_folder(tmp_path, name, with_stream_weights=True):
    """A model folder whose matrices are N(0, 1 / fan_in) (projections keep the size of their input, attention scores
    are far from uniform), norm weights 1 + N(0, 0.1), sinks spread over a few units either way (some heads give
    half their weight away, others nothing), blending weights between 0.2 and 0.8, and stream weights near the
    identity but with every entry of `mix` far enough from 0 and 1 to show."""
    import torch
    from tuff_b200.config.registry import config_from_dict
    from tuff_b200.models.model import Model
    from tuff_b200.weights import write_safetensors
    cfg, seed = CONFIGS[name]
    arch, typed = config_from_dict(cfg, name)
    rng = np.random.default_rng(seed)
    tensors = []
    for tname, decl in sorted(Model(arch.model_spec(typed)).expected_tensors().items()):
        last = tname.rsplit(".", 1)[-1]
        if last == "sink":
            a = 2.0 * rng.normal(size=decl.shape)
        elif last == "vmix":
            a = rng.uniform(0.2, 0.8, size=decl.shape)
        elif ".hc" in tname and last == "mix":
            a = np.eye(decl.shape[0]) * 0.8 + 0.25 * rng.normal(size=decl.shape)
        elif ".hc" in tname:
            a = 1.0 + 0.3 * rng.normal(size=decl.shape)
        elif decl.init == "norm":
            a = 1.0 + 0.1 * rng.normal(size=decl.shape)
        elif tname == "embed":
            a = rng.normal(size=decl.shape)
        else:
            a = rng.normal(size=decl.shape) / np.sqrt(decl.shape[-1])
        tensors.append((tname, torch.tensor(a, dtype=torch.float32).to(torch.bfloat16)))
    folder = str(tmp_path / name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
