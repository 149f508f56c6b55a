"""Fidinex as a `ModelSpec`.

A pre-norm decoder (`rmsnorm`) over a token embedding, with a head tied to the embedding table.  The layers
keep several residual streams (block `hyper_connections`; a model without the streams' weights runs the
ordinary `prenorm` block).  A layer's mixer is one of

  "attention"          `gqa_attention` without position encoding: q and k RMS-normed per head with a learned
                       weight, a query temperature that grows with the position, a learned sink per head, and
                       values blended with those of the first layer that blends (`v_mix`),
  "latent_attention"   `latent_attention`: keys and values expanded from one cached latent vector per token,
                       a rotated key part shared by all heads, a learned sink per head,

and its feed-forward is dense with a squared-relu activation (`relu2_mlp`) or absent.

Checkpoint tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.{up,down}`,
`l<i>.hc<q>.{in,out,mix}` for sublayer q = 1 (mixer), 2 (feed-forward), `final.norm`.
"""
from __future__ import annotations

from ..config.fidinex import ARCHITECTURE, FidinexConfig, SinkAttention
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec


def _mixer(d, eps, m, p, v_role):
    if isinstance(m, SinkAttention):
        names = {"q_proj": p + "q", "k_proj": p + "k", "v_proj": p + "v", "out_proj": p + "o",
                 "q_layernorm": p + "q.norm", "k_layernorm": p + "k.norm", "sink": p + "sink", "vmix": p + "vmix"}
        return PartSpec("gqa_attention",
                        dict(d_model=d, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                             qk_norm_eps=eps, position_encoding=None, scale=m.scale, sink="learned",
                             q_temp=None if m.q_temp is None else (m.q_temp.coef, m.q_temp.every),
                             v_mix=v_role, unused_vmix_weight=v_role is None), names)
    return PartSpec("latent_attention",
                    dict(d_model=d, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_head_dim=m.vdim, kv_rank=m.kv_rank,
                         rot_base=m.rot_base, rot_dims=m.rot_dims, scale=m.scale, norm_eps=eps, sink="learned"),
                    {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                     "sink": p + "sink", "o": p + "o"})


def fidinex_spec(cfg: FidinexConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    seen_source = False
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        has_ff = l.mlp is not None
        v_role = None
        if isinstance(l.mixer, SinkAttention) and l.mixer.v_mix:
            v_role = "blend" if seen_source else "source"      # the first such layer gives its values to the others
            seen_source = True
        if cfg.hyper:
            names = {}
            for q in (("1", "2") if has_ff else ("1",)):
                names.update({"in" + q: f"{p}hc{q}.in", "out" + q: f"{p}hc{q}.out", "mix" + q: f"{p}hc{q}.mix"})
            block = PartSpec("hyper_connections", dict(streams=cfg.streams, has_ffn=has_ff), names)
        else:
            block = PartSpec("prenorm")
        layers.append(LayerSpec(
            mixer=_mixer(d, eps, l.mixer, p + "mix.", v_role),
            ffn=PartSpec("relu2_mlp", dict(d_model=d, ffn_dim=l.mlp.ff), {"up": p + "mlp.up", "down": p + "mlp.down"}) if has_ff else None,
            mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": p + "norm1"}),
            ffn_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": p + "norm2"}) if has_ff else None,
            block=block))
    return ModelSpec(
        architecture=ARCHITECTURE, d_model=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, d_model=d), {"weight": "embed"}),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": "final.norm"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, d_model=d), {"weight": "embed"}))


def refine_config(cfg: FidinexConfig, shapes: dict) -> FidinexConfig:
    return cfg.refine(shapes)
