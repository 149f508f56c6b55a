"""What needs no GPU of the Fidinex design: reading its configuration, the model description and its tensor
names, what its mixers ask of the cache manager, and the plain implementation against closed forms."""
import copy
import json
import math

import numpy as np
import pytest

import plain_fidinex as plain
from tiny_fidinex import CONFIGS, FID_A, FID_B, FID_C, FID_D
from tuff_b200.cache import CacheManager
from tuff_b200.config import ConfigError, config_from_dict
from tuff_b200.models.model import Model
from tuff_b200.parts.base import PagedKVNeed


def test_config_round_trip_and_description():
    for name, (raw, _) in CONFIGS.items():
        arch, cfg = config_from_dict(raw, name)
        assert arch.name == "Fidinex" and cfg == arch.parse_config(arch.config_to_dict(cfg), name)
        assert len(cfg.layers) == len(raw["layers"]) and cfg.vocab == raw["vocab"] and cfg.streams == raw.get("streams")
    _, cfg = config_from_dict(FID_A, "a")
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.q_temp is None and not cfg.layers[2].mixer.v_mix
    assert cfg.layers[1].mixer.q_temp.every == 7 and cfg.layers[0].mixer.kv_rank == 20 and cfg.layers[0].mixer.rot_base == 100.0
    assert cfg.hyper and not config_from_dict(FID_C, "c")[1].hyper


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "dims"), (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 1, "mlp", "kind"), "experts", "kind"), (("layers", 1, "mixer", "q_temp", "every"), 0, "every"),
    (("norm", "eps"), "x", "eps"), (("width",), None, "width"), (("layers",), [], "layers"), (("streams",), 9, "streams"),
    (("layers", 3, "mixer", "vdim"), 24, "vdim")])
def test_config_errors_name_the_key(path, value, word):
    raw = copy.deepcopy(FID_A)
    node = raw
    for p in path[:-1]:
        node = node[p]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw, "cfg")
    assert word in str(e.value)


def test_model_description_and_tensor_names():
    arch, cfg = config_from_dict(FID_A, "a")
    model = Model(arch.model_spec(cfg))
    exp = model.expected_tensors()
    assert exp["l0.mix.q"].shape == (3 * (16 + 8), 80) and exp["l0.mix.dkv"].shape == (20 + 8, 80)
    assert exp["l0.mix.dkv.norm"].shape == (20,) and exp["l0.mix.uk"].shape == (3 * 16, 20) and exp["l0.mix.uv"].shape == (3 * 24, 20)
    assert exp["l0.mix.o"].shape == (80, 3 * 24) and exp["l0.mix.sink"].shape == (3,)
    assert exp["l1.mix.q"].shape == (4 * 24, 80) and exp["l1.mix.k"].shape == (2 * 24, 80) and exp["l1.mix.v"].shape == (2 * 40, 80)
    assert exp["l1.mix.q.norm"].shape == (24,) and exp["l1.mix.vmix"].shape == () and exp["l1.mix.o"].shape == (80, 4 * 40)
    assert exp["l1.hc1.mix"].shape == (2, 2) and exp["l1.hc2.in"].shape == (2,) and exp["l0.mlp.up"].shape == (96, 80)
    assert "l2.norm2" not in exp and "l2.mlp.up" not in exp and "l2.hc2.in" not in exp and "l2.hc1.out" in exp
    assert exp["l2.mix.vmix"].optional and not exp["l3.mix.vmix"].optional
    assert exp["embed"].shape == (301, 80) and exp["final.norm"].shape == (80,) and "head" not in exp
    needs = model.storage_needs()
    assert needs[0] == PagedKVNeed(1, 28, v_head_dim=20, values_in_keys=True)
    assert needs[1] == PagedKVNeed(2, 24, v_head_dim=40) and needs[2] == PagedKVNeed(2, 32)
    # which layer gives its values and which take them
    roles = [l.mixer.v_mix if hasattr(l.mixer, "v_mix") else None for l in model.layers]
    assert roles == [None, "source", None, "blend", "blend"]
    # no streams: the ordinary layer
    arch, cfg = config_from_dict(FID_C, "c")
    assert not any(".hc" in n for n in Model(arch.model_spec(cfg)).expected_tensors())


def test_streams_without_their_weights_fall_back_to_one_residual(tmp_path):
    import torch
    from tuff_b200.config.registry import load_config
    from tuff_b200.weights import write_safetensors
    with open(tmp_path / "config.json", "w") as f:
        json.dump(FID_B, f)
    write_safetensors(str(tmp_path / "model.safetensors"), [("embed", torch.zeros(257, 64, dtype=torch.bfloat16))])
    arch, cfg = load_config(str(tmp_path))
    assert cfg.streams == 1 and not cfg.hyper
    assert not any(".hc" in n for n in Model(arch.model_spec(cfg)).expected_tensors())


def test_latent_rows_are_paged_like_keys():
    """A mixer whose values lie inside its keys asks for pages of one key/value head as wide as a latent row; mixers
    of equal shape share a group of pages and its table."""
    arch, cfg = config_from_dict(FID_D, "d")
    needs = Model(arch.model_spec(cfg)).storage_needs()
    cm = CacheManager(needs, page_size=8, max_tokens=64, max_requests=2)
    assert needs[1] == PagedKVNeed(1, 200 + 64, v_head_dim=200, values_in_keys=True)
    assert len(cm.groups) == 4 - 1 + (needs[2] != needs[3])
    rc = cm.open("a")
    cm.reserve(rc, 20); cm.commit(rc, 20); cm.check()
    assert all(sum(p != -1 for p in t) == 3 for t in rc.tables)
    cm.close(rc); cm.check()
    assert all(g.pool.n_held == 0 for g in cm.groups)


def test_plain_sink_softmax_temperature_and_rotation():
    p = plain.sink_softmax(np.zeros((1, 4)), 0.0, np.array([[True, True, False, False]]))
    assert np.allclose(p, [[1 / 3, 1 / 3, 0, 0]])
    p = plain.sink_softmax(np.array([[2.0, 2.0]]), 2.0 + math.log(2.0), np.array([[True, True]]))
    assert np.allclose(p, [[0.25, 0.25]])
    p = plain.sink_softmax(np.array([[800.0, 0.0]]), -800.0, np.array([[True, True]]))          # no overflow either way
    assert np.allclose(p, [[1.0, 0.0]])
    t = plain.query_temperature([0, 5, 6, 12, 13, 20], 0.5, 7)
    assert np.allclose(t, [1, 1, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(4)])
    x = np.zeros((2, 1, 6)); x[:, 0, 0] = 1.0; x[:, 0, 3] = 2.0; x[:, 0, 5] = 7.0
    base = 16.0
    y = plain.rotate_pairs(x, [0, 1], base, 4)
    assert np.allclose(y[0], x[0])
    a0, a1 = 1.0, base ** (-2.0 / 4)
    assert np.allclose(y[1, 0], [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 0, 7.0])


def test_plain_streams_reduce_to_the_ordinary_layer():
    """One stream with in = out = mix = 1 is x + f(norm(x)); with several, `mix` is read [from, to]."""
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 8)); nw = 1 + 0.1 * rng.normal(size=8)
    f = lambda h: np.tanh(h) * 3.0
    one = plain.hyper_sublayer(x[None], {"p.in": np.ones(1), "p.out": np.ones(1), "p.mix": np.ones((1, 1))}, "p.", f, nw, 1e-5)
    assert np.allclose(one[0], x + f(plain.rms_norm(x, nw, 1e-5)))
    xs = rng.normal(size=(2, 5, 8))
    w = {"p.in": np.array([1.0, 0.0]), "p.out": np.array([0.0, 1.0]), "p.mix": np.array([[0.0, 1.0], [0.0, 0.0]])}
    two = plain.hyper_sublayer(xs, w, "p.", f, nw, 1e-5)
    assert np.allclose(two[0], 0.0) and np.allclose(two[1], xs[0] + f(plain.rms_norm(xs[0], nw, 1e-5)))


def test_plain_latent_attention_is_attention_over_expanded_keys():
    """The latent mixer against ordinary attention on keys and values written out per head."""
    rng = np.random.default_rng(1)
    T, d, H, dim, rd, vd, rank = 9, 12, 2, 4, 2, 3, 5
    m = dict(heads=H, dim=dim, rot_dim=rd, vdim=vd, kv_rank=rank, scale=0.7, rot=dict(base=10.0, dims=rd))
    w = {"x.q": rng.normal(size=(H * (dim + rd), d)), "x.dkv": rng.normal(size=(rank + rd, d)), "x.dkv.norm": rng.normal(size=rank),
         "x.uk": rng.normal(size=(H * dim, rank)), "x.uv": rng.normal(size=(H * vd, rank)), "x.sink": np.array([0.3, -1.0]),
         "x.o": rng.normal(size=(d, H * vd))}
    h = rng.normal(size=(T, d))
    got = plain.latent_attention(h, w, "x.", m, 1e-5)
    dkv = h @ w["x.dkv"].T
    c = plain.rms_norm(dkv[:, :rank], w["x.dkv.norm"], 1e-5)
    out = np.zeros((T, H, vd))
    for t in range(T):
        for a in range(H):
            q = (w["x.q"] @ h[t])[a * (dim + rd):(a + 1) * (dim + rd)]
            qr = plain.rotate_pairs(q[None, None, dim:], [t], 10.0, rd)[0, 0]
            s = []
            for j in range(t + 1):
                kr = plain.rotate_pairs(dkv[j][None, None, rank:], [j], 10.0, rd)[0, 0]
                s.append((q[:dim] @ (w["x.uk"][a * dim:(a + 1) * dim] @ c[j]) + qr @ kr) * 0.7)
            e = np.exp(np.array(s))
            p = e / (e.sum() + math.exp(w["x.sink"][a]))
            out[t, a] = sum(p[j] * (w["x.uv"][a * vd:(a + 1) * vd] @ c[j]) for j in range(t + 1))
    assert np.allclose(got, out.reshape(T, -1) @ w["x.o"].T)
