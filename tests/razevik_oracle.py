"""A slow float64 restatement of the Razevik design, one function per mechanism, written from its equations.  It takes a
configuration dictionary and a name -> tensor mapping and shares no code with the package: whole sequences, every key
and value formed explicitly per head, experts evaluated one token at a time.

Notation: h is a sublayer's input [T, W]; linear weights are [out, in] and act as W h.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def _w(sd: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return sd[name].to(F64)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def latent_of(h: torch.Tensor, sd, p: str, eps: float) -> torch.Tensor:
    """The key/value latent of every token: c = rms_norm(W_dkv h) [T, kv_rank] (what a cache holds)."""
    return rms_norm(h @ _w(sd, p + "dkv").T, _w(sd, p + "dkv.norm"), eps)


def latent_attention(h: torch.Tensor, c: torch.Tensor, sd, p: str, m: Dict[str, Any], eps: float) -> torch.Tensor:
    """Causal softmax attention whose keys and values are per-head expansions of the latents c [T, kv_rank] (this layer's
    own or another layer's), queries through a normed latent of their own, a sigmoid gate per head, then W_o."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ _w(sd, p + "dq").T, _w(sd, p + "dq.norm"), eps)
    q = (cq @ _w(sd, p + "uq").T).view(T, H, D)
    k = (c @ _w(sd, p + "uk").T).view(T, H, D)
    v = (c @ _w(sd, p + "uv").T).view(T, H, V)
    gate = torch.sigmoid(h @ _w(sd, p + "g").T)                       # [T, H]
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        for a in range(H):
            s = (k[: i + 1, a] @ q[i, a]) * m["scale"]
            w = torch.softmax(s, 0)
            out[i, a] = (w[:, None] * v[: i + 1, a]).sum(0) * gate[i, a]
    return out.reshape(T, H * V) @ _w(sd, p + "o").T


def dense_ff(h: torch.Tensor, sd, p: str) -> torch.Tensor:
    return relu_squared(h @ _w(sd, p + "up").T) @ _w(sd, p + "down").T


def route(h: torch.Tensor, sd, p: str, r: Dict[str, Any]) -> Tuple[List[List[int]], torch.Tensor]:
    """Per token: the `top` experts by sigmoid score + correction among the experts of the `keep` best groups (a group
    is ranked by the sum of its two largest corrected scores), and their uncorrected scores normalised to sum 1."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ _w(sd, p + "router").T)
    corr = _w(sd, p + "correction") if (p + "correction") in sd else torch.zeros(E, dtype=F64)
    chosen, weights = [], torch.zeros(h.shape[0], top, dtype=F64)
    for t in range(h.shape[0]):
        choice = (s[t] + corr).tolist()
        allowed = set(range(E))
        g = r.get("groups")
        if g:
            size = E // g["count"]
            rank = []
            for j in range(g["count"]):
                members = sorted(choice[j * size:(j + 1) * size], reverse=True)
                rank.append((-sum(members[:2]), j))
            kept = [j for _, j in sorted(rank)[: g["keep"]]]
            allowed = {e for j in kept for e in range(j * size, (j + 1) * size)}
        order = sorted(allowed, key=lambda e: (-choice[e], e))[:top]
        chosen.append(order)
        raw = torch.stack([s[t, e] for e in order])
        weights[t] = raw / (raw.sum() + 1e-20)
    return chosen, weights


def expert(h: torch.Tensor, sd, p: str) -> torch.Tensor:
    return gelu_erf(h @ _w(sd, p + "up").T) @ _w(sd, p + "down").T


def moe_ff(h: torch.Tensor, sd, p: str, f: Dict[str, Any]) -> torch.Tensor:
    chosen, weights = route(h, sd, p, f["router"])
    y = torch.zeros(h.shape[0], h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for c, e in enumerate(chosen[t]):
            y[t] += weights[t, c] * expert(h[t:t + 1], sd, f"{p}e{e}.")[0]
    if f.get("shared"):
        y = y + torch.sigmoid(h @ _w(sd, p + "shared.sg").T) * expert(h, sd, p + "shared.")
    return y


def token_side(x: torch.Tensor, tokens: torch.Tensor, i: int, sd, cfg: Dict[str, Any]) -> torch.Tensor:
    """x + m * rms_norm(W_proj (gelu_tanh(W_gate x) * e)) with e the layer's slice of the tokens' side embedding."""
    d = cfg["token_side"]["dim"]
    p = f"l{i}.side."
    e = _w(sd, "side.embed")[tokens][:, i * d:(i + 1) * d]
    y = (gelu_tanh(x @ _w(sd, p + "gate").T) * e) @ _w(sd, p + "proj").T
    return x + cfg["residual_mult"] * rms_norm(y, _w(sd, p + "norm"), cfg["norm"]["eps"])


def forward(cfg: Dict[str, Any], sd: Dict[str, torch.Tensor], tokens) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """logits [T, vocab] of a whole sequence and the residual stream after every layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    T, eps, m = tokens.numel(), cfg["norm"]["eps"], cfg["residual_mult"]
    x = _w(sd, "embed")[tokens] + _w(sd, "pos")[:T]
    latents: Dict[int, torch.Tensor] = {}
    taps = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert L["type"] == "latent_attention"
        h1 = rms_norm(x, _w(sd, p + "norm1"), eps)
        src = L["mixer"].get("kv_from")
        if src is None:
            latents[i] = latent_of(h1, sd, p + "mix.", eps)
            src = i
        y = latent_attention(h1, latents[src], sd, p + "mix.", L["mixer"], eps)
        f = L.get("mlp")
        if f:
            h2 = rms_norm(x, _w(sd, p + "norm2"), eps)
            y = y + (dense_ff(h2, sd, p + "mlp.") if f["kind"] == "dense" else moe_ff(h2, sd, p + "mlp.", f))
        x = x + m * y
        if cfg.get("token_side"):
            x = token_side(x, tokens, i, sd, cfg)
        taps.append(x)
    logits = rms_norm(x, _w(sd, "final.norm"), eps) @ _w(sd, "head").T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, taps


# ---- small configurations and random weights for the tests ------------------------------------------------------------
def make_config(width=48, vocab=61, layers=("own", "shared", "own"), heads=3, dim=8, vdim=12, kv_rank=16, q_rank=24,
                scale=0.3, ff=20, experts=6, top=2, groups=(3, 2), shared_ff=28, dense_ff=40, side_dim=6, mult=0.7,
                softcap=9.0, eps=1e-5, max_positions=512) -> Dict[str, Any]:
    """layers: "own" (latent attention with its own latents + mixture of experts), "shared" (reads the latents of the
    nearest earlier "own" layer), "dense" (own latents + dense feed-forward), "bare" (own latents, no feed-forward), or a
    dictionary {"kind": one of these, **overrides of heads / dim / vdim / kv_rank / q_rank / scale / kv_from / mlp}."""
    out, last_own = [], None
    for i, spec in enumerate(layers):
        spec = {"kind": spec} if isinstance(spec, str) else dict(spec)
        kind = spec.pop("kind")
        mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
        moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
        if groups:
            moe["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
        if shared_ff:
            moe["shared"] = {"ff": shared_ff}
        mlp = {"own": moe, "shared": moe, "dense": {"kind": "dense", "ff": dense_ff}, "bare": None}[kind]
        if "mlp" in spec:
            mlp = spec.pop("mlp")
        if kind == "shared":
            mixer["kv_from"] = last_own
        mixer.update(spec)
        if "kv_from" in mixer and mixer["kv_from"] is not None:
            mixer["kv_rank"] = out[mixer["kv_from"]]["mixer"]["kv_rank"]
        else:
            last_own = i
        out.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Razevik", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps},
           "residual_mult": mult, "layers": out}
    if side_dim:
        cfg["token_side"] = {"dim": side_dim}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def random_weights(cfg: Dict[str, Any], seed: int = 0, head_gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors under the checkpoint's names."""
    g = torch.Generator().manual_seed(seed)
    W, n = cfg["width"], len(cfg["layers"])

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg["vocab"], W), "pos": rnd(cfg["max_positions"], W, std=0.5),
          "head": rnd(cfg["vocab"], W, std=head_gain * W ** -0.5), "final.norm": rnd(W, std=0.1, mean=1.0)}
    d = (cfg.get("token_side") or {}).get("dim", 0)
    if d:
        sd["side.embed"] = rnd(cfg["vocab"], d * n)
    s = W ** -0.5
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, D, V, R, Q = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        sd[p + "norm1"] = rnd(W, std=0.1, mean=1.0)
        sd[p + "mix.dq"], sd[p + "mix.dq.norm"], sd[p + "mix.uq"] = rnd(Q, W, std=s), rnd(Q, std=0.1, mean=1.0), rnd(H * D, Q, std=2 * Q ** -0.5)
        if m.get("kv_from") is None:
            sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = rnd(R, W, std=s), rnd(R, std=0.1, mean=1.0)
        sd[p + "mix.uk"], sd[p + "mix.uv"] = rnd(H * D, R, std=2 * R ** -0.5), rnd(H * V, R, std=R ** -0.5)
        sd[p + "mix.g"], sd[p + "mix.o"] = rnd(H, W, std=2 * s), rnd(W, H * V, std=(H * V) ** -0.5)
        f = L["mlp"]
        if f:
            sd[p + "norm2"] = rnd(W, std=0.1, mean=1.0)
            if f["kind"] == "dense":
                sd[p + "mlp.up"], sd[p + "mlp.down"] = rnd(f["ff"], W, std=s), rnd(W, f["ff"], std=f["ff"] ** -0.5)
            else:
                E, ffe = f["router"]["experts"], f["expert"]["ff"]
                sd[p + "mlp.router"], sd[p + "mlp.correction"] = rnd(E, W, std=2 * s), rnd(E, std=0.3)
                for e in range(E):
                    sd[p + f"mlp.e{e}.up"], sd[p + f"mlp.e{e}.down"] = rnd(ffe, W, std=s), rnd(W, ffe, std=ffe ** -0.5)
                if f.get("shared"):
                    fs = f["shared"]["ff"]
                    sd[p + "mlp.shared.up"], sd[p + "mlp.shared.down"] = rnd(fs, W, std=s), rnd(W, fs, std=fs ** -0.5)
                    sd[p + "mlp.shared.sg"] = rnd(1, W, std=2 * s)
        if d:
            sd[p + "side.gate"], sd[p + "side.proj"], sd[p + "side.norm"] = rnd(d, W, std=s), rnd(W, d, std=d ** -0.5), rnd(W, std=0.1, mean=1.0)
    return sd
