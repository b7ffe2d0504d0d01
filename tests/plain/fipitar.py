"""Plain, slow implementation of the Fipitar decoder: whole sequences, no cache, no state carried between calls, one
function per mechanism.

It is the oracle the engine is compared with and shares no code with ``mashbox_b200``: it reads config.json's keys
itself (a dict) and works on CPU tensors in float64.

The design, in this file's notation.  T tokens at positions 0 .. T-1, width D, rms(x) = x / sqrt(mean(x^2) + eps),
ln(x; w, b) = (x - mean) / sqrt(var + eps) w + b.

  stream   : x = E[token];  per layer  x <- x + ln1(mixer(x));  x <- x + ln2(ff(x)) when the layer has a feed-forward
             (the sublayers read the stream as it is; only what they return is normed);  logits = W_head ln_f(x)
  gla      : q = Wq h dim^-1/2, k = Wk h (heads x dim), v = Wv h (heads x vdim);
             a = sigmoid(Wa2 Wa1 h + ba)^(1/tau) (heads x dim: one decay per head and key channel);
             per head  S <- diag(a) S + k v^T;  o = S^T q;  out = Wo (concat_h(rms(o_h) n) * silu(Wg h))
  latent   : cq = rms(Wdq h) nq;  q_h = Wuq cq = [u_h (dim) | r_h (rot_dim)];  Wdkv h = [c' (kv_rank) | kr (rot_dim)],
             c = rms(c') nkv;  key of head h: [Wuk_h c | kr], value Wuv_h c;  r_h and kr are rotated (adjacent pairs,
             frequencies bent between two wavelengths, cos and sin times a gain);
             s_ij = scale (u_i . Wuk_h c_j + r_i . kr_j), j <= i;  p_ij = e^s_ij / (e^sink_h + sum_j e^s_ij);
             out = Wo concat_h(sum_j p_ij Wuv_h c_j)
  capped   : q, k (kv heads shared by runs of query heads), v = W h;  q, k <- rms(.) n per head;  the first R dims of
             q and k rotated (dim i with dim i + R/2);  s = cap tanh(scale q.k / cap);  p_ij = e^s_ij / (1 + sum_j e^s_ij);
             out = Wo concat_h(sigmoid(Wg h)_h sum_j p_ij v_j)
  ssd      : Win h = [z | x | B | C | dt];  (x, B, C) <- silu(conv(x, B, C) + bias), a causal filter per channel;
             dt <- softplus(dt + dt_bias);  per head (its B, C from group h // (heads / groups))
             S <- exp(-exp(A_h) dt) S + dt B x^T;  y = S^T C + D_h x;
             out = Wo (rms over each of `norm_groups` equal parts of (y * silu(z)) times n)
  pair     : left_scale capped(h) + right_scale ssd(h)
  ff       : g = min(Wg h, L), u = clamp(Wu h, -L, L);  Wd (g sigmoid(1.702 g) (u + 1))
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def layer_norm(x, w, b, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def frequencies(rot):
    """-> (one angle per position step for every rotated pair, the gain on cos and sin)"""
    R = int(rot["dims"])
    base = float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / R) for i in range(R // 2)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):       # the (fractional) pair index whose wavelength makes `turns` turns over the original length
        return R * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), R - 1)
    ramp = torch.clamp((torch.arange(R // 2, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, layout):
    """x (T, heads, dim): the first rot["dims"] values of every head turn by position * frequency; layout "halves"
    pairs value i with value i + dims/2, "adjacent" pairs value 2i with value 2i + 1"""
    if not rot or not rot.get("dims"):
        return x
    R = int(rot["dims"])
    f, gain = frequencies(rot)
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(a) * gain)[:, None, :], (torch.sin(a) * gain)[:, None, :]
    if layout == "halves":
        u, v = x[..., :R // 2], x[..., R // 2:R]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., R:]], -1)
    u, v = x[..., 0:R:2], x[..., 1:R:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], -1).reshape(*x.shape[:-1], R)
    return torch.cat([turned, x[..., R:]], -1)


def gla(W, p, m, h, eps):
    T = h.shape[0]
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, dim)
    v = (h @ W[p + "v"].T).view(T, H, vdim)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    a = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).view(T, H, dim)
    S = torch.zeros(H, dim, vdim, dtype=F64)
    o = torch.zeros(T, H, vdim, dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = (rms(o, eps) * W[p + "norm"]).reshape(T, H * vdim) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def softmax_with_sink(s, sink):
    """s (..., T, T) with -inf where a key is not seen; sink (...) broadcast over the rows: one more term in the
    denominator that has no value"""
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[..., None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[..., None] - m))


def causal(T):
    return torch.tril(torch.ones(T, T, dtype=torch.bool))


def latent_attention(W, p, m, h, eps):
    T = h.shape[0]
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    rd, rank = int(m.get("rot_dim") or 0), int(m["kv_rank"])
    pos = torch.arange(T)
    cq = rms(h @ W[p + "dq"].T, eps, W[p + "dq.norm"])
    q = (cq @ W[p + "uq"].T).view(T, H, dim + rd)
    low = h @ W[p + "dkv"].T
    c = rms(low[:, :rank], eps, W[p + "dkv.norm"])
    k = (c @ W[p + "uk"].T).view(T, H, dim)
    v = (c @ W[p + "uv"].T).view(T, H, vdim)
    s = torch.einsum("ihd,jhd->hij", q[..., :dim], k)
    if rd:
        qr = rotate(q[..., dim:], pos, m.get("rot"), "adjacent")
        kr = rotate(low[:, None, rank:], pos, m.get("rot"), "adjacent")[:, 0]
        s = s + torch.einsum("ihd,jd->hij", qr, kr)
    s = (s * float(m["scale"])).masked_fill(~causal(T), -math.inf)
    w = softmax_with_sink(s, W[p + "sink"].to(F64)[:, None].expand(H, T))
    return torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * vdim) @ W[p + "o"].T


def capped_attention(W, p, m, h, eps):
    T = h.shape[0]
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    G = int(m.get("kv_heads") or H)
    pos = torch.arange(T)
    q = rotate(rms((h @ W[p + "q"].T).view(T, H, dim), eps, W[p + "q.norm"]), pos, m.get("rot"), "halves")
    k = rotate(rms((h @ W[p + "k"].T).view(T, G, dim), eps, W[p + "k.norm"]), pos, m.get("rot"), "halves")
    v = (h @ W[p + "v"].T).view(T, G, vdim)
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    s = s.masked_fill(~causal(T), -math.inf)
    w = softmax_with_sink(s, torch.zeros(H, T, dtype=F64))
    o = torch.einsum("hij,jhd->ihd", w, v) * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * vdim) @ W[p + "o"].T


def causal_conv(u, w, b):
    """u (T, C), w (C, taps) whose last column meets the current token, zeros before the start"""
    T, taps = u.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    return sum(pad[j:j + T] * w[:, j] for j in range(taps)) + b


def ssd(W, p, m, h, eps):
    T = h.shape[0]
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m.get("groups") or 1)
    inner, parts = H * P, int(m.get("norm_groups") or 1)
    rows = h @ W[p + "in"].T
    z, xbc, dt = rows[:, :inner], rows[:, inner:2 * inner + 2 * G * N], rows[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, 1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, 1)
    dt = softplus(dt + W[p + "dt_bias"])
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + W[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def pair(W, p, m, h, eps):
    return (float(m.get("left_scale", 1.0)) * capped_attention(W, p + "left.", m["left"], h, eps)
            + float(m.get("right_scale", 1.0)) * ssd(W, p + "right.", m["right"], h, eps))


def feed_forward(W, p, f, h):
    L = float(f["limit"])
    g = torch.clamp(h @ W[p + "gate"].T, max=L)
    u = torch.clamp(h @ W[p + "up"].T, -L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


MIXERS = {"gla": gla, "latent_attention": latent_attention, "parallel": pair}


def forward(cfg, W, tokens, after_layers=None):
    """config.json as a dict, tensors by stored name (any float dtype), token ids -> float64 logits (T, vocab);
    after_layers: a list that receives the stream after every layer"""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](W, p + "mix.", layer["mixer"], x, eps)
        x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(W, p + "mlp.", layer["mlp"], x)
            x = x + layer_norm(y, W[p + "norm2"], W[p + "norm2.b"], eps)
        if after_layers is not None:
            after_layers.append(x.clone())
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
