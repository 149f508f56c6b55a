"""Fidinex on the GPU against the plain implementation (tests/plain_fidinex.py): every mechanism alone,
whole models replayed in four ways, pages used again, keys far away and at page borders, sinks, long
decoding past several periods of the query temperature, and generation through the engine's own entry point."""
import io
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_fidinex as plain
import traces
from test_gpu_parts import DT, bind_random, dev, f64, make_ctx, run_part_in_portions
from tiny import random_tokens
from tiny_fidinex import CONFIGS, make_folder
from tuff_b200.cache import CacheManager

pytestmark = pytest.mark.gpu

# Root mean square of the difference of a logits row (mean taken off) over that of the row itself.
ROW_TOL = {"float32": 2e-4, "bfloat16": 6e-2}
LENGTHS = {"fid_a": (70, 45, 97, 130, 66), "fid_b": (83, 40, 129, 65, 100), "fid_c": (150, 64, 37, 200, 129),
           "fid_d": (120, 51, 33, 160, 101), "fid_e": (300, 129, 517, 64, 200), "fid_f": (190, 64, 131, 260, 77)}
PAGE = {"fid_a": 16, "fid_b": 4, "fid_c": 64, "fid_d": 8, "fid_e": 32, "fid_f": 16}


def row_error(got, ref):
    d = got - ref
    d = d - d.mean()
    return float(np.sqrt((d * d).mean()) / max(1e-9, np.sqrt(((ref - ref.mean()) ** 2).mean())))


class Plain:
    def __init__(self, folder):
        self.cfg, self.w = plain.load(folder)

    def forward(self, tokens, collect=None):
        return plain.forward(self.cfg, self.w, tokens, collect)


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("fidinex")
    out = {}
    for name in CONFIGS:
        folder = make_folder(base, name)
        vocab = CONFIGS[name][0]["vocab"]
        reqs = {f"r{i}": random_tokens(vocab, n, 10 * i + len(name)) for i, n in enumerate(LENGTHS[name])}
        p = Plain(folder)
        out[name] = (folder, reqs, {rid: p.forward(t) for rid, t in reqs.items()})
    return out


def run_trace(folder, dtype, steps, tmp_path, page_size, max_tokens=None):
    from tuff_b200.engine.replay import replay
    from tuff_b200.engine.runner import ModelRunner
    n = max_tokens or traces.tokens_needed(steps, round_to=max(64, page_size))
    runner = ModelRunner(folder, dtype=dtype, max_tokens=n, page_size=page_size, max_requests=4)
    runner.cache.owners = {}
    log = io.StringIO()
    replay(runner, io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), str(tmp_path), report=log)
    assert log.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    runner.cache.check()
    assert not runner.cache.live
    return runner


def logits_by_place(out_dir, wanted, vocab):
    out = {}
    for step, rows in wanted.items():
        got = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for i, place in enumerate(rows):
            out[place] = got[i].copy()
    return out


def compare(out_dir, wanted, expect, vocab, dtype, what):
    for (rid, pos), got in logits_by_place(out_dir, wanted, vocab).items():
        err = row_error(got, expect[rid][pos])
        assert err <= ROW_TOL[dtype], f"{what} {dtype}: request {rid} position {pos}: error {err:.3g}"


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "tail_decoded", "portions", "mixed"])
def test_replay_modes(models, tmp_path, name, dtype, mode):
    folder, reqs, expect = models[name]
    steps, wanted = getattr(traces, mode)(reqs)
    runner = run_trace(folder, dtype, steps, tmp_path, PAGE[name])
    compare(str(tmp_path), wanted, expect, CONFIGS[name][0]["vocab"], dtype, f"{name} {mode}")
    if mode == "mixed":
        reused = [k for k, who in runner.cache.owners.items() if len(set(who)) > 1]
        assert len(reused) >= 1, runner.cache.owners


@pytest.mark.parametrize("name", ["fid_a", "fid_d"])
def test_float32_logits_do_not_depend_on_the_cut(models, tmp_path, name):
    """Every sum of the 32-bit path runs in an order that the sizes alone decide: a (request, position) has
    the same logits, bit for bit, whole, with its tail decoded, in portions, and mixed with others."""
    folder, reqs, _ = models[name]
    vocab = CONFIGS[name][0]["vocab"]
    seen = None
    for mode in ("whole", "tail_decoded", "portions", "mixed"):
        steps, wanted = getattr(traces, mode)(reqs)
        out = tmp_path / mode
        run_trace(folder, "float32", steps, out, PAGE[name])
        got = logits_by_place(str(out), wanted, vocab)
        if seen is None:
            seen = got
        else:
            for place, row in got.items():
                assert np.array_equal(row, seen[place]), (mode, place, np.abs(row - seen[place]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["fid_a", "fid_c"])
def test_layers_one_by_one(models, dtype, name):
    """The stream (the sum of the streams, where there are several) after every layer, against the plain
    implementation's."""
    from tuff_b200.engine.batch import StepEntry, layout_entries, to_device
    from tuff_b200.engine.runner import ModelRunner
    folder, reqs, _ = models[name]
    toks = reqs["r1"]
    ref = []
    Plain(folder).forward(toks, ref)
    runner = ModelRunner(folder, dtype=dtype, max_tokens=128, page_size=8, max_requests=2)
    rc = runner.open("x")
    runner.cache.reserve(rc, len(toks))
    ctx = to_device(layout_entries([StepEntry(rc, toks, [])], runner.cache), runner.device, runner.dtype)
    m = runner.model
    x = m.embedding.forward(ctx)
    for i, e in enumerate(m.schedule):
        layer = m.layers[e.layer]
        layer.block.forward(ctx, x, layer, runner.cache.storages[e.storage], False)
        now = layer.block.finish(ctx, x)           # folds what is pending; the next layer goes on from the streams
        err = np.abs(f64(now) - ref[i]).max()
        assert err <= (3e-5 if dtype == "float32" else 6e-2) * (i + 1) * max(1.0, np.abs(ref[i]).max()), (i, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_entry_point(models, name, dtype):
    from tuff_b200 import Engine, SamplingParams
    folder = models[name][0]
    vocab = CONFIGS[name][0]["vocab"]
    prompts = [random_tokens(vocab, n, 40 + n) for n in (7, 13, 1, 30, 5)]
    eng = Engine(folder, dtype=dtype, ctx_size=128, max_tokens=256, page_size=8, max_batched_tokens=16, max_running=3)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    assert [len(o) for o in outs] == [12] * 5
    p = Plain(folder)
    margin = 1e-3 if dtype == "float32" else 0.3
    for prompt, out in zip(prompts, outs):
        ref = p.forward(prompt + out)
        for i, tok in enumerate(out):
            row = ref[len(prompt) + i - 1]
            assert row.max() - row[tok] <= margin * max(1.0, row.std()), (i, tok, int(row.argmax()), row.max() - row[tok])
    eng.runner.cache.check()
    assert not eng.runner.cache.live


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["fid_a", "fid_c"])
def test_long_decoding(models, tmp_path, name, dtype):
    """A short prompt, then 250 tokens one by one: the query temperature passes many of its periods (3, 7, 16 and
    50 positions), the keys run over many pages."""
    folder = models[name][0]
    vocab = CONFIGS[name][0]["vocab"]
    toks = random_tokens(vocab, 253, 5)
    steps, wanted = traces.tail_decoded({"long": toks}, tail=250)
    run_trace(folder, dtype, steps, tmp_path, page_size=8, max_tokens=256)
    compare(str(tmp_path), wanted, {"long": Plain(folder).forward(toks)}, vocab, dtype, "long decoding")


@pytest.mark.parametrize("name", ["fid_a", "fid_b"])
def test_first_tokens_and_single_token_requests(models, tmp_path, name):
    folder, _, _ = models[name]
    vocab = CONFIGS[name][0]["vocab"]
    reqs = {"one": random_tokens(vocab, 1, 1), "two": random_tokens(vocab, 2, 2), "three": random_tokens(vocab, 3, 3)}
    expect = {rid: Plain(folder).forward(t) for rid, t in reqs.items()}
    for mode in ("whole", "portions"):
        steps, wanted = getattr(traces, mode)(reqs, *(((1, 1, 1),) if mode == "portions" else ()))
        run_trace(folder, "float32", steps, tmp_path / mode, 4)
        compare(str(tmp_path / mode), wanted, expect, vocab, "float32", f"first tokens {mode}")


def test_pages_are_used_again_in_a_small_pool(models, tmp_path):
    """Five requests one after the other in a pool that holds one of them: every page serves several requests,
    and what the earlier ones left in them does not show."""
    folder, reqs, expect = models["fid_b"]
    steps, wanted = traces.portions(reqs, sizes=(9, 2, 30, 1))
    runner = run_trace(folder, "float32", steps, tmp_path, 4, max_tokens=192)
    compare(str(tmp_path), wanted, expect, CONFIGS["fid_b"][0]["vocab"], "float32", "small pool")
    assert max(len(set(who)) for who in runner.cache.owners.values()) >= 3


# ------------------------------------------------------------------ mechanisms alone
def _plain_names(w, p="x."):
    names = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o", "q_layernorm": "q.norm", "k_layernorm": "k.norm",
             "sink": "sink", "vmix": "vmix"}
    return {p + names.get(n, n): a for n, a in w.items()}


class _SourceThenBlend:
    """Two attention layers of one step: the first leaves its values for the second, whose output is what counts."""

    def __init__(self, first, second, cm):
        self.first, self.second, self.cm = first, second, cm

    def forward(self, ctx, storage, x, res):
        self.first.forward(ctx, self.cm.storages[0], x, torch.zeros_like(res))
        self.second.forward(ctx, self.cm.storages[1], x, res)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,vd,page,q_temp", [(4, 2, 24, 40, 4, (0.5, 7)), (3, 3, 16, 8, 8, None), (6, 1, 48, 64, 16, (0.3, 64)),
                                                   (4, 2, 64, 64, 16, (0.4, 5)), (2, 1, 128, 128, 8, (1.0, 3)), (8, 2, 64, 64, 64, None)])
def test_sink_attention_part_with_blended_values(dtype, H, G, hd, vd, page, q_temp):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(H + hd + vd)
    d, eps, scale = 64, 1e-5, 0.3
    common = dict(d_model=d, num_heads=H, num_kv_heads=G, head_dim=hd, v_head_dim=vd, qk_norm_eps=eps, position_encoding=None,
                  scale=scale, sink="learned", q_temp=q_temp)
    first = MIXERS.build(PartSpec("gqa_attention", dict(v_mix="source", **common)))
    second = MIXERS.build(PartSpec("gqa_attention", dict(v_mix="blend", **common)))
    w1 = bind_random(first, dtype, rng, std=0.3)
    w2 = {}
    for n, decl in second.weight_decls().items():
        a = {"sink": 2.0 * rng.normal(size=decl.shape), "vmix": np.array(0.35)}.get(
            n, 1 + 0.1 * rng.normal(size=decl.shape) if decl.init == "norm" else 0.3 * rng.normal(size=decl.shape))
        w2[n] = dev(a, torch.float32 if decl.role == "vector" else DT[dtype])
    second.bind(dict(w2), DT[dtype])
    w2 = {n: f64(t) for n, t in w2.items()}
    cm = CacheManager([first.cache_need(), second.cache_need()], page_size=page, max_tokens=512, max_requests=3, dtype=DT[dtype],
                      device="cuda:0")
    for part in (first, second):
        part.reserve("cuda:0", 256, 512)
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (150, 6, 70)]
    got = run_part_in_portions(_SourceThenBlend(first, second, cm), cm, None, dtype, hs, cuts=(3, 1, 7, 2, 1, 30, 64))
    m = dict(heads=H, kv_heads=G, dim=hd, vdim=vd, scale=scale, v_mix=True, q_temp=dict(coef=q_temp[0], every=q_temp[1]) if q_temp else None)
    for g, h in zip(got, hs):
        _, v_first = plain.attention(h, _plain_names(w1), "x.", m, eps)
        ref, _ = plain.attention(h, _plain_names(w2), "x.", m, eps, v_first)
        alone, _ = plain.attention(h, _plain_names(w2), "x.", dict(m, v_mix=False), eps)
        assert np.abs(ref - alone).max() > 0.05                                   # the blend shows
        assert np.abs(g - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())
    cm.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dim,rd,vd,rank,page", [(3, 16, 8, 24, 20, 4), (2, 24, 4, 16, 40, 8), (5, 8, 16, 12, 12, 16),
                                                   (4, 32, 32, 32, 64, 64), (2, 40, 64, 20, 200, 8), (16, 64, 32, 64, 128, 32),
                                                   (1, 16, 0, 16, 32, 4), (4, 32, 32, 64, 64, 16), (2, 64, 64, 128, 256, 64),
                                                   (3, 96, 32, 128, 136, 8), (16, 64, 64, 128, 512, 32)])
def test_latent_attention_part(dtype, H, dim, rd, vd, rank, page):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(H + dim + rank)
    d, eps, base = 72, 1e-5, 50.0
    scale = 1.5 * min(1.0, (64.0 / (rank + rd)) ** 0.5)       # scores of a few units whatever the width of the latent
    part = MIXERS.build(PartSpec("latent_attention", dict(d_model=d, num_heads=H, head_dim=dim, rot_dim=rd, v_head_dim=vd,
                                                          kv_rank=rank, rot_base=base, rot_dims=rd, scale=scale, norm_eps=eps)))
    w = bind_random(part, dtype, rng, std=0.12)
    w["sink"] = 2.0 * rng.normal(size=H)
    part.sinks.copy_(dev(w["sink"]))
    part.reserve("cuda:0", 256, 512)
    cm = CacheManager([part.cache_need()], page_size=page, max_tokens=512, max_requests=3, dtype=DT[dtype], device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (140, 5, 67)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(3, 1, 7, 2, 1, 30, 64))
    m = dict(heads=H, dim=dim, rot_dim=rd, vdim=vd, kv_rank=rank, scale=scale, rot=dict(base=base, dims=rd))
    names = {"dkv_norm": "dkv.norm"}
    pw = {"x." + names.get(n, n): a for n, a in w.items()}
    for g, h in zip(got, hs):
        ref = plain.latent_attention(h, pw, "x.", m, eps)
        assert np.abs(g - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())
    cm.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,d,F", [(1, 64, 128), (5, 80, 96), (40, 100, 72), (300, 256, 512), (16, 256, 1024)])
def test_relu_squared_feed_forward_part(dtype, T, d, F):
    from tuff_b200.engine.batch import StepContext
    from tuff_b200.parts import FEED_FORWARDS, PartSpec
    rng = np.random.default_rng(T + F)
    part = FEED_FORWARDS.build(PartSpec("relu2_mlp", dict(d_model=d, ffn_dim=F)))
    w = bind_random(part, dtype, rng, std=0.2)
    h = dev(rng.normal(size=(T, d)), DT[dtype])
    res0 = rng.normal(size=(T, d))
    res = dev(res0)
    part.forward(None, h, res)
    z = f64(h) @ w["up"].T
    if dtype == "bfloat16":
        z = f64(dev(z, torch.bfloat16))
    ref = res0 + plain.relu_squared_mlp(f64(h), {"x.up": w["up"], "x.down": w["down"]}, "x.")
    assert np.abs(f64(res) - ref).max() <= (3e-5 if dtype == "float32" else 4e-2) * max(1, np.abs(ref).max())
    assert (plain.relu_squared_mlp(f64(h), {"x.up": w["up"], "x.down": np.eye(F)}, "x.") == 0).mean() > 0.3     # the negative half is cut


@pytest.mark.parametrize("S,T,d", [(1, 3, 64), (2, 7, 80), (3, 130, 256), (4, 33, 100), (8, 2, 48)])
def test_streams_step_kernel(S, T, d):
    """The kernel between two sublayers: the update that one sublayer left, then the read-out and norm of the next,
    against the plain implementation's sublayer (with the sublayer's function given as the y already computed)."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(S * T)
    xs = rng.normal(size=(S, T, d)); y = rng.normal(size=(T, d))
    w = {"x.in": rng.normal(size=S), "x.out": rng.normal(size=S), "x.mix": rng.normal(size=(S, S))}
    nw, eps = 1 + 0.1 * rng.normal(size=d), 1e-3
    new = plain.hyper_sublayer(xs, w, "x.", lambda h: y, nw, eps)
    assert S == 1 or np.abs(new - np.einsum("ts,sij->tij", w["x.mix"], xs) - w["x.out"][:, None, None] * y).max() > 0.1   # [from, to] shows
    in2 = rng.normal(size=S)
    u_ref = np.tensordot(in2, new, axes=(0, 0))
    X, yd = dev(xs), dev(y)
    u = torch.empty(T, d, device="cuda")
    for hdt in (torch.float32, torch.bfloat16):
        X, yd = dev(xs), dev(y)
        h = torch.empty(T, d, device="cuda", dtype=hdt)
        ops.hc_step(X, y=yd, mix=dev(w["x.mix"]), out_w=dev(w["x.out"]), in_w=dev(in2), norm_w=dev(nw), eps=eps, h_out=h, u_out=u)
        assert np.abs(f64(X) - new).max() < 2e-5 and np.abs(f64(u) - u_ref).max() < 2e-5 and float(yd.abs().max()) == 0.0
        href = plain.rms_norm(u_ref, nw, eps)
        assert np.abs(f64(h) - href).max() <= (2e-5 if hdt == torch.float32 else 2e-2) * max(1, np.abs(href).max())
    # the start (every stream is the embedding's output) and the end (the plain sum of the streams)
    x0 = rng.normal(size=(T, d))
    ops.hc_step(X, x_init=dev(x0), in_w=dev(in2), u_out=u)
    assert np.abs(f64(X) - x0[None]).max() < 1e-6 and np.abs(f64(u) - in2.sum() * x0).max() < 2e-5
    ops.hc_step(X, u_out=u)
    assert np.abs(f64(u) - S * x0).max() < 2e-5


def test_query_temperature_at_the_edges_of_its_periods():
    from tuff_b200.kernels import ops
    H, G, hd = 2, 1, 16
    for coef, every in ((0.3, 64), (1.0, 3), (0.5, 1), (0.2, 1000)):
        pos = np.array(sorted({0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 2 * every, 7 * every - 1, 4095} - {-1}))
        T = len(pos)
        x = np.random.default_rng(every).normal(size=(T, (H + 2 * G) * hd))
        qk = dev(x).contiguous()
        ops.qk_norm_rope_write(qk, None, None, None, dev(pos, torch.int32), torch.zeros(T, dtype=torch.int32, device="cuda"), None,
                               None, None, H, G, hd, 0, 0.0, write_kv=False, q_temp=(coef, every))
        ref = x.copy()
        ref[:, : H * hd] *= plain.query_temperature(pos, coef, every)[:, None]
        assert np.abs(f64(qk) - ref).max() < 1e-5 * np.abs(ref).max()
        t = plain.query_temperature([every - 2, every - 1], coef, every)
        assert every == 1 or (t[0] == 1.0 and abs(t[1] - (1 + coef * math.log(2.0))) < 1e-12)


# ------------------------------------------------------------------ keys that stand out, sinks
def _paged(k, v, page, G, kd, vd, dtype, values_in_keys=False):
    """Pages handed out in descending order, so that a page's number says nothing about its place."""
    T = k.shape[0]
    n_pages = (T + page - 1) // page
    kp = torch.zeros(n_pages + 1, G, page, kd, device="cuda", dtype=dtype)
    vp = None if values_in_keys else torch.zeros(n_pages + 1, G, page, vd, device="cuda", dtype=dtype)
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").flip(0).reshape(1, -1).contiguous()
    pages = table[0].long()
    for t in range(T):
        kp[pages[t // page], :, t % page] = dev(k[t], dtype).view(G, kd)
        if vp is not None:
            vp[pages[t // page], :, t % page] = dev(v[t], dtype).view(G, vd)
    return kp, vp, table


def _attend(q, kp, vp, table, out, H, G, kd, cuts, **kw):
    from tuff_b200.kernels import ops
    T = q.shape[0]
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    rows = torch.zeros(T, dtype=torch.int32, device="cuda")
    p = 0
    for n in cuts:
        n = min(n, T - p)
        if n <= 0:
            break
        single = n == 1
        ops.paged_attention(q[p:p + n], kp, vp, table, positions[p:p + n], rows[:n], out[p:p + n], H, G, kd, 1.0,
                            all_single=single, max_seq_len=T, single_prefix=0,
                            cu_q=None if single else torch.tensor([0, n], dtype=torch.int32, device="cuda"), **kw)
        p += n
    assert p == T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kd,vd,page,in_keys", [(32, 48, 4, False), (48, 64, 16, False), (64, 64, 16, False), (128, 128, 64, False),
                                                 (96, 64, 16, True), (40, 24, 8, True), (160, 128, 32, True)])
def test_one_far_key_among_hundreds_and_learned_sinks(dtype, kd, vd, page, in_keys):
    """One key whose score is far above all others, at the first place, at a page's last and first place and
    hundreds of places back: every later query of the heads that ask for it returns its value, scaled by what
    the head's sink takes; the place before the key does not see it.  In portions and token by token."""
    H, G, T = 4, (1 if in_keys else 2), 400
    rng = np.random.default_rng(kd + page)
    dt = DT[dtype]
    sinks = np.array([-30.0, 3.0, 0.0, 1.5])            # head 0 gives nothing away
    for key_at in (0, page - 1, page, 3 * page, 137):
        k = f64(dev(0.1 * rng.normal(size=(T, G * kd)), dt)); q = f64(dev(0.1 * rng.normal(size=(T, H * kd)), dt))
        col = kd - 1                                     # a column that is not part of the values when they lie in the keys
        k[key_at, :kd] = 0.0; k[key_at, col] = 6.0
        if in_keys:                                      # one key/value head: a value is the key's first vd elements
            k[key_at, :vd] = np.arange(vd) % 7 - 3.0
            v = k[:, :vd]
        else:
            v = f64(dev(rng.normal(size=(T, G * vd)), dt))
        q[:, col] = 5.0; q[:, kd + col] = 5.0           # heads 0 and 1 (key/value head 0) ask for it
        kp, vp, table = _paged(k, v, page, G, kd, vd, dt, in_keys)
        ref = np.zeros((T, H, vd))
        vis = plain.causal_mask(T)
        for a in range(H):
            g = a // (H // G)
            ref[:, a] = plain.sink_softmax(q[:, a * kd:(a + 1) * kd] @ k[:, g * kd:(g + 1) * kd].T, sinks[a], vis) @ v[:, g * vd:(g + 1) * vd]
        qd = dev(q, dt)
        for cuts in ((128, 7, 1, 1, 100, 2, 161), (1,) * 30 + (2, 368)):
            out = torch.zeros(T, H * vd, device="cuda", dtype=dt)
            _attend(qd, kp, vp, table, out, H, G, kd, cuts, sink=dev(sinks), v_head_dim=vd, values_in_keys=in_keys)
            got = f64(out).reshape(T, H, vd)
            assert np.abs(got - ref).max() <= (2e-4 if dtype == "float32" else 3e-2), (key_at, cuts[:2], np.abs(got - ref).max())
        vk = v[key_at, :vd]
        assert np.abs(got[T - 1, 0] - vk).max() < 3e-2 * max(1, np.abs(vk).max())          # seen from 260 places on, whole
        if key_at > 0:
            assert np.abs(got[key_at - 1, 0] - vk).max() > 0.2                             # not before it exists
    # a sink that is as large as the standing-out score takes half
    share = plain.sink_softmax(np.array([[30.0]]), 30.0, np.array([[True]]))
    assert abs(share[0, 0] - 0.5) < 1e-12


@pytest.mark.parametrize("H,rank,rd,page,splits", [(4, 64, 32, 16, 0), (16, 128, 64, 64, 3), (20, 72, 8, 8, 5), (33, 512, 64, 32, 0),
                                                   (1, 32, 0, 4, 32), (7, 200, 24, 16, 2)])
def test_latent_decode_kernel_far_keys_and_sinks(monkeypatch, H, rank, rd, page, splits):
    """Single tokens of two requests over a latent cache, every head in one pass: one cached row whose score stands
    out for two heads (at the first place, at a page's edges, at a tile's edges, far back), a sink that takes a head's
    whole weight and sinks that take a share; contexts of 1 to 400 rows, with the keys cut into 1 to 32 slices
    (more slices than tiles too).  Against the sums written out in float64."""
    from tuff_b200.kernels import ops
    if splits:
        monkeypatch.setenv("TUFF_LATENT_SPLITS", str(splits))
    hl, T = rank + rd, 400
    rng = np.random.default_rng(H * rank + page)
    bf = torch.bfloat16
    assert ops.latent_decode_supported(torch.empty(1, dtype=bf), torch.empty(1, dtype=bf), H, rank, rd)
    sinks = rng.normal(size=H); sinks[0] = 40.0; sinks[-1] = -30.0
    hot = [h for h in (1, H - 1) if h < H and h > 0] or [0]
    for key_at in (0, page - 1, page, 63, 64, 137):
        rows = f64(dev(0.1 * rng.normal(size=(2, T, hl)), bf))
        rows[0, key_at] = 0.0; rows[0, key_at, hl - 1] = 6.0; rows[0, key_at, :rank] = np.arange(rank) % 5 - 2.0
        if rd == 0:                                   # no rotated part: the score's column lies inside the values
            rows[0, key_at, :rank] = 0.0; rows[0, key_at, rank - 1] = 6.0
        n_pages = -(-T // page)
        kp = torch.zeros(2 * n_pages + 1, 1, page, hl, device="cuda", dtype=bf)
        table = torch.arange(2 * n_pages, dtype=torch.int32, device="cuda").flip(0).reshape(2, n_pages).contiguous()
        for r in range(2):
            full = torch.zeros(n_pages * page, hl, device="cuda", dtype=bf)
            full[:T] = dev(rows[r], bf)
            kp[table[r].long(), 0] = full.view(n_pages, page, hl)
        places = sorted({0, 1, key_at, max(0, key_at - 1), key_at + 1, 62, 63, 64, 65, 127, 128, 200, 399})
        pos = np.array([q for q in places for _ in range(2)]); row_of = np.array([0, 1] * len(places))
        n = len(pos)
        ql = f64(dev(0.1 * rng.normal(size=(n, H, hl)), bf))
        for h in hot:
            ql[:, h, hl - 1] = 5.0
        out = torch.full((n, H, rank), 7.0, device="cuda", dtype=bf)
        ops.latent_decode(dev(ql, bf), kp, table, dev(pos, torch.int32), dev(row_of, torch.int32), out, H, rank, rd, 0.9,
                          sink=dev(sinks), max_seq_len=T)
        got = f64(out)
        for i in range(n):
            keys = rows[row_of[i], : pos[i] + 1]
            for h in range(H):
                sc = 0.9 * keys @ ql[i, h]
                wts = plain.sink_softmax(sc[None, :], sinks[h], np.ones((1, len(sc)), bool))[0]
                ref = wts @ keys[:, :rank]
                assert np.abs(got[i, h] - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max()), (key_at, i, h)
        if H > 1:
            assert np.abs(got[:, 0]).max() < 1e-6                               # the sink of head 0 keeps everything
        seen = [i for i in range(n) if row_of[i] == 0 and pos[i] >= key_at]
        if rd and H > 1 and sinks[hot[-1]] < 10:
            for i in seen:                                                       # the far row alone, whole, for the heads that ask
                assert np.abs(got[i, hot[-1]] - rows[0, key_at, :rank]).max() < 0.1


@pytest.mark.parametrize("T,H,K,N", [(1, 3, 16, 20), (8, 16, 64, 128), (9, 5, 130, 7), (64, 2, 512, 64), (128, 1, 24, 33), (17, 2, 1024, 70),
                                     (3, 4, 5, 64)])
def test_head_linear_of_few_rows(T, H, K, N):
    """A matrix per head applied to views with strides (heads inside wider rows), few tokens: the one-warp-per-column kernel."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(T + K)
    bf = torch.bfloat16
    wide = dev(rng.normal(size=(T, H, K + 6)), bf)
    w = dev(rng.normal(size=(H, N, K)) / math.sqrt(K), bf)
    outw = torch.zeros(T, H, N + 2, device="cuda", dtype=bf)
    ref = np.einsum("thk,hnk->thn", f64(wide[:, :, 2:2 + K]), f64(w))
    for wt in (None, w.transpose(1, 2).contiguous()):        # a warp per column; a thread per column of the transposed matrices
        outw.zero_()
        ops.head_linear(wide[:, :, 2:2 + K], w, outw[:, :, :N], wt=wt)
        assert np.abs(f64(outw[:, :, :N]) - ref).max() <= 1e-2 * max(1.0, np.abs(ref).max())
        assert float(outw[:, :, N:].abs().max()) == 0.0


@pytest.mark.parametrize("hd,vd,page", [(16, 16, 4), (64, 64, 16), (128, 128, 32), (24, 40, 8)])
def test_learned_sinks_take_their_share(hd, vd, page):
    """Scores of zero over n keys and sinks ln(1), ln(3), -inf-like: the weights are 1 / (n + e^sink)."""
    from tuff_b200.kernels import ops
    H, G, T = 3, 1, 70
    dt = torch.bfloat16 if hd >= 64 else torch.float32
    v = f64(dev(np.random.default_rng(8).normal(size=(T, vd)), dt))
    kp, vp, table = _paged(np.zeros((T, hd)), v, page, G, hd, vd, dt)
    sinks = np.array([0.0, math.log(3.0), -40.0])
    for cuts in ((T,), (1,) * T, (3, 1, 64, 2)):
        out = torch.empty(T, H * vd, device="cuda", dtype=dt)
        _attend(torch.zeros(T, H * hd, device="cuda", dtype=dt), kp, vp, table, out, H, G, hd, cuts, sink=dev(sinks), v_head_dim=vd)
        got = f64(out).reshape(T, H, vd)
        for a, extra in enumerate((1.0, 3.0, 0.0)):
            ref = np.cumsum(v, axis=0) / (np.arange(T) + 1.0 + extra)[:, None]
            assert np.abs(got[:, a] - ref).max() < (1e-5 if dt == torch.float32 else 2e-2), (cuts[:2], a)


def test_trace_run_program_and_command_line(models, tmp_path):
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, reqs, expect = models["fid_b"]
    vocab = CONFIGS["fid_b"][0]["vocab"]
    steps, wanted = traces.mixed(reqs)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", str(traces.tokens_needed(steps))], input=text, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        compare(str(out), wanted, expect, vocab, dtype, "trace_run")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "tuff"), "--model", folder, "--prompt-ids", "5 9 200 31", "-n", "6",
                        "--dump-tokens", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.split()]
    ref = Plain(folder).forward([5, 9, 200, 31] + ids[-6:])
    for i, tok in enumerate(ids[-6:]):
        assert ref[3 + i].max() - ref[3 + i][tok] < 1e-3
