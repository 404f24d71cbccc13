"""Razevik adapter: a text-only decoder-only LM on ``HybridEngine`` (hybrid_engine.py) whose blocks run their mixer and
their feed-forward in parallel on two RMS norms of the same fp32 stream, x += m * (mixer(n1 x) + ff(n2 x)), followed by a
per-token side input (a slice of a second embedding of the token, gated by the stream, projected, RMS-normed and added).
Learned absolute positions are added to the embedding; there is no rotation anywhere.

  * mixer: latent attention -- queries through a normed latent, keys and values per-head expansions of one normed
    key/value latent per token, which is all the layer caches; a layer may read an earlier layer's cached latents instead
    of projecting its own (``kv_from``); one sigmoid gate per head.
  * feed-forward: none, dense (down(relu(up h)^2)), or a mixture of experts of the form down(gelu(up h)) behind a
    sigmoid router (choice by score + correction among the best groups of neighbouring experts, weights = the chosen
    scores normalised) plus a shared expert times a per-token sigmoid gate.
  * output: RMS norm, head, soft cap cap * tanh(logits / cap).

Everything a model of this design can vary is read from its ``config.json``; serving (worker, scheduler, pages, sampler,
command lines) is what ``BobavikModel`` set up for hybrid-engine designs.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from .._lib import VoxB200Error
from ..hybrid_engine import DenseMLPConfig, HybridConfig, HybridLayerConfig, LatentAttentionConfig, MoEConfig
from .bobavik import BobavikModel


def razevik_config(c: Dict[str, Any]) -> HybridConfig:
    """config.json -> HybridConfig.  Keys: ``width``, ``vocab``, ``max_positions``, ``norm.eps``, ``residual_mult``,
    ``token_side.dim`` (optional), ``logit_softcap`` (optional) and ``layers``: per layer ``type`` (latent_attention),
    ``mixer`` {heads, dim, vdim, kv_rank, q_rank, scale, kv_from?} and ``mlp``: null, {kind: dense, ff} or {kind: moe,
    expert.ff, router.{experts, top, groups.{count, keep}?}, shared.ff?}."""
    layers = []
    for i, L in enumerate(c["layers"]):
        if L["type"] != "latent_attention":
            raise VoxB200Error(f"layer {i}: unknown mixer type '{L['type']}'")
        m = L["mixer"]
        kv_from = m.get("kv_from")
        mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), int(m["kv_rank"]),
                                      int(m["q_rank"]), float(m.get("scale", int(m["dim"]) ** -0.5)),
                                      None if kv_from is None else int(kv_from))
        f = L.get("mlp")
        mlp = None
        if f:
            kind = f.get("kind", "dense")
            if kind == "dense":
                mlp = DenseMLPConfig(int(f["ff"]), "relu2")
            elif kind == "moe":
                r, g, sh = f["router"], f["router"].get("groups") or {}, f.get("shared") or {}
                mlp = MoEConfig(int(r["experts"]), int(r["top"]), int(f["expert"]["ff"]), int(sh.get("ff", 0) or 0),
                                act="gelu", router="sigmoid", groups=int(g.get("count", 0) or 0),
                                groups_keep=int(g.get("keep", 0) or 0), shared_gate=bool(sh.get("ff")))
                if mlp.groups > 1 and (mlp.experts % mlp.groups or not 1 <= mlp.groups_keep <= mlp.groups or
                                       mlp.groups_keep * (mlp.experts // mlp.groups) < mlp.top):
                    raise VoxB200Error(f"layer {i}: {mlp.groups} groups (keep {mlp.groups_keep}) do not fit {mlp.experts} "
                                       f"experts, top {mlp.top}")
            else:
                raise VoxB200Error(f"layer {i}: unknown feed-forward kind '{kind}'")
        layers.append(HybridLayerConfig("latent", mixer, mlp))
    side = c.get("token_side") or {}
    return HybridConfig(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), 1.0, layers, block="parallel",
                        norm="rmsnorm", residual_mult=float(c.get("residual_mult", 1.0)),
                        positions=int(c["max_positions"]), side_dim=int(side.get("dim", 0) or 0),
                        logit_softcap=float(c.get("logit_softcap", 0.0) or 0.0))


def synthetic_state_dict(cfg: HybridConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights with the checkpoint's names (bf16), generated on ``device``."""
    g = torch.Generator(device=device).manual_seed(seed)
    W, n = cfg.width, len(cfg.layers)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg.vocab, W), "pos": rnd(cfg.positions, W, std=0.5), "head": rnd(cfg.vocab, W, std=W ** -0.5),
          "final.norm": rnd(W, std=0.1, mean=1.0)}
    if cfg.side_dim:
        sd["side.embed"] = rnd(cfg.vocab, cfg.side_dim * n)
    s = W ** -0.5
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        sd[p + "norm1"] = rnd(W, std=0.1, mean=1.0)
        sd[p + "mix.dq"], sd[p + "mix.dq.norm"] = rnd(m.q_rank, W, std=s), rnd(m.q_rank, std=0.1, mean=1.0)
        sd[p + "mix.uq"] = rnd(m.heads * m.dim, m.q_rank, std=m.q_rank ** -0.5)
        if m.kv_from is None:
            sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = rnd(m.kv_rank, W, std=s), rnd(m.kv_rank, std=0.1, mean=1.0)
        sd[p + "mix.uk"] = rnd(m.heads * m.dim, m.kv_rank, std=m.kv_rank ** -0.5)
        sd[p + "mix.uv"] = rnd(m.heads * m.vdim, m.kv_rank, std=m.kv_rank ** -0.5)
        sd[p + "mix.g"], sd[p + "mix.o"] = rnd(m.heads, W, std=s), rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        f = L.mlp
        if f is not None:
            sd[p + "norm2"] = rnd(W, std=0.1, mean=1.0)
        if isinstance(f, DenseMLPConfig):
            sd[p + "mlp.up"], sd[p + "mlp.down"] = rnd(f.ff, W, std=s), rnd(W, f.ff, std=f.ff ** -0.5)
        elif f is not None:
            sd[p + "mlp.router"], sd[p + "mlp.correction"] = rnd(f.experts, W, std=s), rnd(f.experts, std=0.2)
            for e in range(f.experts):
                sd[p + f"mlp.e{e}.up"], sd[p + f"mlp.e{e}.down"] = rnd(f.ff, W, std=s), rnd(W, f.ff, std=f.ff ** -0.5)
            if f.shared_ff:
                sd[p + "mlp.shared.up"] = rnd(f.shared_ff, W, std=s)
                sd[p + "mlp.shared.down"] = rnd(W, f.shared_ff, std=f.shared_ff ** -0.5)
                sd[p + "mlp.shared.sg"] = rnd(1, W, std=s)
        if cfg.side_dim:
            sd[p + "side.gate"], sd[p + "side.proj"] = rnd(cfg.side_dim, W, std=s), rnd(W, cfg.side_dim, std=cfg.side_dim ** -0.5)
            sd[p + "side.norm"] = rnd(W, std=0.1, mean=1.0)
    return sd


class RazevikModel(BobavikModel):
    design = "Razevik"
    synthetic_name = "razevik-synthetic"
    has_recurrent_state = False

    @staticmethod
    def read_config(config: Dict[str, Any]) -> HybridConfig:
        return razevik_config(config)

    @staticmethod
    def synthetic_weights(cfg: HybridConfig, seed: int, device) -> Dict[str, torch.Tensor]:
        return synthetic_state_dict(cfg, seed, device)
