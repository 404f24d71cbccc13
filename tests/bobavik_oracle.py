"""Plain, slow float64 implementation of the Bobavik design for the tests: one function per mechanism, whole sequences at a
time, token loops where the definition is a recurrence.  Shares no code with vox_serve_b200.

Notation: x [T, W] residual stream; for a mixer with input h:  attention  q = Wq h, k = Wk h, v = Wv h, rotate pairs
(2i, 2i+1) of the first `rot.dims` dims of q and k by angle pos * f_i, score_ij = scale * q_i . k_j for i - window < j <= i,
out = softmax(score) v, gated by sigmoid(Wg h);  lightning  q, k, v = silu(W. h), S_t = decay_h S_(t-1) + k_t v_t^T,
o_t = S_t^T q_t, rms-normed over all heads, gated;  feed-forward  top-k experts by router logits, softmax over the chosen
logits, plus a shared expert.  Every sublayer: x += LN_after(sublayer(LN_before(x))).
"""
import math

import torch

F64 = torch.float64


def make_config(width=64, vocab=96, layers=("attention", "lightning"), heads=4, kv_heads=2, dim=16, vdim=8, window=8,
                rot_dims=8, rot_base=10000.0, scaling=(4.0, 1.0, 4.0, 64), scale=0.25, v_mix=True, lin_heads=2, lin_dim=16,
                lin_vdim=16, decay=(0.9, 0.6), experts=4, top=2, ff=24, shared_ff=40, eps=1e-5, logit_scale=0.75, mlp=True):
    """A config.json dictionary; `layers` is the order of mixer types (an entry may be a dict of overrides with 'type')."""
    out = []
    for L in layers:
        o = {"type": L} if isinstance(L, str) else dict(L)
        kind = o.pop("type")
        if kind == "attention":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
            if window:
                mixer["mask"] = {"size": window}
            if rot_dims:
                mixer["rot"] = {"dims": rot_dims, "base": rot_base}
                if scaling:
                    mixer["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        else:
            mixer = {"heads": lin_heads, "dim": lin_dim, "vdim": lin_vdim, "decay": list(decay)}
        has_mlp = o.pop("mlp", mlp)
        mixer.update(o)
        f = None
        if has_mlp:
            f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
            if shared_ff:
                f["shared"] = {"ff": shared_ff}
        out.append({"type": kind, "mixer": mixer, "mlp": f})
    return {"architecture": "Bobavik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": out}


def random_weights(cfg, seed=0, head_gain=1.0):
    """name -> tensor with the checkpoint's names; values are exactly representable in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def r(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    sd = {"embed": r(cfg["vocab"], W), "head": r(cfg["vocab"], W, std=head_gain * W ** -0.5),
          "final.norm": r(W, std=0.1, mean=1.0), "final.norm.b": r(W, std=0.1)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if L["mlp"] else ()):
            sd[p + nm], sd[p + nm + ".b"] = r(W, std=0.1, mean=1.0), r(W, std=0.1)
        s = W ** -0.5
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        G = m.get("kv_heads", H) if L["type"] == "attention" else H
        sd[p + "mix.q"], sd[p + "mix.k"] = r(H * dk, W, std=s), r(G * dk, W, std=s)
        sd[p + "mix.v"], sd[p + "mix.g"] = r(G * dv, W, std=s), r(H * dv, W, std=s)
        sd[p + "mix.o"] = r(W, H * dv, std=(H * dv) ** -0.5)
        if L["type"] == "attention":
            if m.get("v_mix"):
                sd[p + "mix.vmix"] = torch.rand((), generator=g).to(torch.bfloat16)
        else:
            sd[p + "mix.norm"] = r(H * dv, std=0.1, mean=1.0)
        if L["mlp"]:
            f = L["mlp"]
            E = f["router"]["experts"]
            sd[p + "mlp.router"], sd[p + "mlp.router.b"] = r(E, W, std=2 * s), r(E, std=0.3)
            for nm, ff in [(f"e{e}", f["expert"]["ff"]) for e in range(E)] + \
                          ([("shared", f["shared"]["ff"])] if f.get("shared") else []):
                sd[p + f"mlp.{nm}.gate"], sd[p + f"mlp.{nm}.up"] = r(ff, W, std=s), r(ff, W, std=s)
                sd[p + f"mlp.{nm}.down"] = r(W, ff, std=ff ** -0.5)
    return sd


# ---- mechanisms ---------------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    n = rot["dims"]
    out = []
    for i in range(n // 2):
        f = rot["base"] ** (-2.0 * i / n)
        sc = rot.get("scaling")
        if sc:
            wavelength = 2 * math.pi / f
            if wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wavelength >= sc["original"] / sc["high"]:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x, positions, rot):
    """x [T, heads, dim]; dims 2i, 2i+1 (i < rot.dims / 2) form a pair."""
    n = rot["dims"]
    ang = positions.to(F64)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    y = x.clone()
    y[..., 0:n:2] = a * c - b * s
    y[..., 1:n:2] = b * c + a * s
    return y


def window_attention(q, k, v, scale, window):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] at positions 0..T-1 -> [T, H, dv]; window 0 = all earlier positions."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, 0) @ v[lo:i + 1, g]
    return out


def decay_attention(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv] -> [T, H, dv], the recurrence token by token from a zero state."""
    T, H, dk = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        S = torch.zeros(dk, v.shape[2], dtype=F64)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router_w, router_b, top):
    z = h @ router_w.T + router_b
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe(h, Wt, p, f):
    idx, wt = route(h, Wt[p + "router"], Wt[p + "router.b"], f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[t, c])
            out[t] += wt[t, c] * gated_expert(h[t], Wt[p + f"e{e}.gate"], Wt[p + f"e{e}.up"], Wt[p + f"e{e}.down"])
    if f.get("shared"):
        out = out + gated_expert(h, Wt[p + "shared.gate"], Wt[p + "shared.up"], Wt[p + "shared.down"])
    return out


# ---- the model ----------------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, layer_outputs=None):
    """tokens: list of ids -> logits [T, vocab] (float64)."""
    Wt = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = Wt["embed"][torch.tensor(tokens)]
    T = x.shape[0]
    pos = torch.arange(T)
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]

        def ln(name, y):
            return layer_norm(y, Wt[p + name], Wt[p + name + ".b"], eps)
        h = ln("norm1", x)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m.get("kv_heads", H)
            q = (h @ Wt[p + "mix.q"].T).view(T, H, dk)
            k = (h @ Wt[p + "mix.k"].T).view(T, G, dk)
            v = (h @ Wt[p + "mix.v"].T).view(T, G, dv)
            if m.get("rot"):
                q, k = rotate_pairs(q, pos, m["rot"]), rotate_pairs(k, pos, m["rot"])
            if m.get("v_mix"):
                if v_first is None:
                    v_first = v
                else:
                    lam = Wt[p + "mix.vmix"]
                    v = (1 - lam) * v + lam * v_first
            o = window_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size", 0))
            o = o.reshape(T, H * dv) * torch.sigmoid(h @ Wt[p + "mix.g"].T)
        else:
            q = silu(h @ Wt[p + "mix.q"].T).view(T, H, dk)
            k = silu(h @ Wt[p + "mix.k"].T).view(T, H, dk)
            v = silu(h @ Wt[p + "mix.v"].T).view(T, H, dv)
            o = decay_attention(q, k, v, m["decay"]).reshape(T, H * dv)
            o = rms_norm(o, eps) * Wt[p + "mix.norm"] * torch.sigmoid(h @ Wt[p + "mix.g"].T)
        x = x + ln("norm1b", o @ Wt[p + "mix.o"].T)
        if L["mlp"]:
            x = x + ln("norm2b", moe(ln("norm2", x), Wt, p + "mlp.", L["mlp"]))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = layer_norm(x, Wt["final.norm"], Wt["final.norm.b"], eps)
    return (x @ Wt["head"].T) * cfg["logit_scale"]


def greedy(cfg, weights, prompt, n_new):
    """prompt + n_new greedy tokens; also the margin (top1 - top2 logit) of every generated token."""
    toks, margins = list(prompt), []
    for _ in range(n_new):
        z = forward(cfg, weights, toks)[-1]
        top = torch.topk(z, 2)
        toks.append(int(top.indices[0]))
        margins.append(float(top.values[0] - top.values[1]))
    return toks[len(prompt):], margins
