"""Plain, slow implementation of the Tosevik decoder: whole sequences, no cache, no state carried between calls, one
function per mechanism.

It is the oracle the engine is compared with and shares no code with ``mashbox_b200``: it reads config.json's keys
itself (a dict) and works on CPU tensors in float64.

The design, in this file's notation.  T tokens at positions 0 .. T-1, width D, rms(x) = x / sqrt(mean(x^2) + eps),
dyt(x; a, w, b) = tanh(a x) w + b (a one number, w and b vectors; no mean, no variance, no eps).

  X_0      = dyt(E[token])                                      the stream before the first layer
  layer i  : y = x + mixer(dyt1(x));  y <- y + ff(dyt2(y)) when the layer has a feed-forward;  X_(i+1) = y;
             what the next layer (or the output) reads is x = sum_(j <= i+1) c_i[j] X_j
  retention: q = Wq h, k = Wk h (heads x dim), v = Wv h (heads x vdim); the first R dims of every head of q and k are
             rotated by p f_i, f_i = base^(-2i/R), dim i with dim i + R/2; k <- k dim^-1/2;
             per head  S <- decay_h S + k v^T;  o = S^T q;  o <- o / rms(o);  out = Wo (concat(o) * silu(Wg h))
  sigmoid attention: q = rms(Wq h) nq, k = rms(Wk h) nk over the WHOLE rows (all heads at once);
             q <- q (1 + coef ln(floor((p + 1) / every) + 1));  v_h <- v_h / rms(v_h);
             weight(i, j) = sigmoid(scale q_i . k_j - slope_h (i - j) + pb_h) for j <= i, slope_h = 2^(-8 (h + 1) / H);
             o_i = sum_j weight(i, j) v_j (no normalisation over the keys);  out = Wo concat(o)
  side by side: out = (rms(left(h)) wl + rms(right(h)) wr) / 2, both mixers reading the same h
  routed feed-forward: s = softmax(Wr h); experts outside the `keep` best of `count` runs of neighbours (a run's worth:
             its largest s) cannot be chosen; the `top` largest s win; out = sum scale s_e expert_e(h)
             + sigmoid(wsg . h) shared(h);  expert(h) = Wd (silu(Wg h) * (Wu h))
  logits   = W_head dyt_final(x)
"""
import math

import torch

F64 = torch.float64


def rms(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def dyt(W, name, x):
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rotate(x, positions, rot):
    """x (T, heads, dim): the first rot["dims"] values of every head turn by position * base^(-2 i / dims)"""
    if not rot or not rot.get("dims"):
        return x
    R = int(rot["dims"])
    half = R // 2
    f = float(rot["base"]) ** (-2.0 * torch.arange(half, dtype=F64) / R)
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:R]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., R:]], -1)


def retention(W, p, m, h, eps, state=None, first=0):
    """h (T, D) -> (T, D); state: None (zeros) or a list of per-head (dim, vdim) matrices that is updated in place;
    first: the position of h's first row"""
    T = h.shape[0]
    H, dim, vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = first + torch.arange(T)
    q = rotate((h @ W[p + "q"].T).view(T, H, dim), pos, m.get("rot"))
    k = rotate((h @ W[p + "k"].T).view(T, H, dim), pos, m.get("rot")) * dim ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, vdim)
    S = state if state is not None else [torch.zeros(dim, vdim, dtype=F64) for _ in range(H)]
    o = torch.zeros(T, H, vdim, dtype=F64)
    for t in range(T):
        for a in range(H):
            S[a] = float(m["decay"][a]) * S[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    o = rms(o, eps).reshape(T, H * vdim) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def sigmoid_attention(W, p, m, h, eps):
    T = h.shape[0]
    H, G, dim, vdim = int(m["heads"]), int(m.get("kv_heads") or m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T, dtype=F64)
    q = rms(h @ W[p + "q"].T, eps, W[p + "q.norm"])
    k = rms(h @ W[p + "k"].T, eps, W[p + "k.norm"]).view(T, G, dim)
    qt = m.get("q_temp")
    if qt:
        q = q * (1.0 + float(qt["coef"]) * torch.log(torch.floor((pos + 1) / int(qt["every"])) + 1.0))[:, None]
    q = q.view(T, H, dim)
    v = rms((h @ W[p + "v"].T).view(T, G, vdim), eps)
    out = torch.zeros(T, H, vdim, dtype=F64)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        z = (q[:, a] @ k[:, g].T) * float(m["scale"]) - slope * dist + W[p + "pb"][a]
        w = torch.where(seen, torch.sigmoid(z), torch.zeros((), dtype=F64))
        out[:, a] = w @ v[:, g]
    return out.reshape(T, H * vdim) @ W[p + "o"].T


def side_by_side(W, p, m, h, eps):
    left = sigmoid_attention(W, p + "left.", m["left"], h, eps)
    right = retention(W, p + "right.", m["right"], h, eps)
    return 0.5 * (rms(left, eps, W[p + "left.out"]) + rms(right, eps, W[p + "right.out"]))


def expert(W, p, h):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def choose(s, top, count=1, keep=1):
    """s (T, E) scores -> (T, top) indexes of the chosen experts, largest first, lower index on ties"""
    T, E = s.shape
    c = s.clone()
    if count > 1 and keep < count:
        worth = c.view(T, count, E // count).max(-1).values
        kept = torch.zeros(T, count, dtype=torch.bool)
        for _ in range(keep):
            at = torch.where(kept, -math.inf, worth).argmax(-1)
            kept[torch.arange(T), at] = True
        c = torch.where(kept.repeat_interleave(E // count, 1), c, torch.full_like(c, -math.inf))
    ids = []
    for _ in range(top):
        at = c.argmax(-1)          # torch returns the first of equal values
        ids.append(at)
        c[torch.arange(T), at] = -math.inf
    return torch.stack(ids, 1)


def routed(W, p, f, h):
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {}
    s = torch.softmax(h @ W[p + "router"].T, -1)
    ids = choose(s, top, int(groups.get("count") or 1), int(groups.get("keep") or groups.get("count") or 1))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in ids[t].tolist():
            out[t] = out[t] + float(r.get("scale", 1.0)) * s[t, e] * expert(W, f"{p}e{e}.", h[t:t + 1])[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * expert(W, p + "shared.", h)
    return out


def forward(cfg, W, tokens, keep_layers=False, keep_results=False):
    """-> logits (T, vocab) float64 (and the stream every layer hands on, when asked; keep_results: instead of it the
    embedding's output and every layer's own result, before the depth average)"""
    W = {k: v.to(F64) if v.is_floating_point() else v for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    t = torch.as_tensor(tokens, dtype=torch.long)
    x = dyt(W, "embed.norm", W["embed"][t])
    history, handed = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dyt(W, p + "norm1", x)
        if layer["type"] == "retention":
            y = x + retention(W, p + "mix.", layer["mixer"], h, eps)
        elif layer["type"] == "parallel":
            y = x + side_by_side(W, p + "mix.", layer["mixer"], h, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            y = y + routed(W, p + "mlp.", layer["mlp"], dyt(W, p + "norm2", y))
        history.append(y)
        x = sum(W[p + "dwa"][j] * history[j] for j in range(i + 2))
        handed.append(x)
    logits = dyt(W, "final.norm", x) @ W["head"].T
    if keep_results:
        return logits, torch.stack(history)
    return (logits, torch.stack(handed)) if keep_layers else logits
