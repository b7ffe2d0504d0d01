"""Small Fipitar configurations with random weights, and the plain implementation's logits for them."""
import functools
import os

import numpy as np
import torch

from mashbox_b200.config.fipitar import (AttentionMixer, DenseFF, FipitarConfig, FipitarLayer, GlaMixer, LatentMixer,
                                         PairMixer, Rotation, SsdMixer)
from tests.plain import fipitar as plain
from tests.plain.llama import read_model


def att(heads, kv, dim, vdim, scale, cap=None, rot=None, base=10000.0):
    return AttentionMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, softcap=cap,
                          rot=Rotation(rot, base) if rot else None)


def ssd(heads, vdim, state, groups=1, parts=1, conv=1):
    return SsdMixer(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=parts, conv=conv)


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None, rot_dims=None):
    rot = Rotation(rot_dims or rot_dim, base, scaling) if rot_dim else None
    return LatentMixer(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale, rot_dim=rot_dim, rot=rot)


def layer(kind, mixer, mlp):
    return FipitarLayer(kind, mixer, mlp)


# P: every size differs from layer to layer where it may.  A recurrent layer first; two query heads per kv head, capped
#    scores, a rotation of part of a head; a convolution of four taps with one group; a latent layer whose frequencies
#    are bent (the bend lies inside its four pairs) and that has no feed-forward; attention without cap and rotation
#    beside a recurrence with two groups and three norm groups
FIP_P = FipitarConfig("Fipitar", width=64, vocab=131, norm_eps=1e-5, layers=(
    layer("gla", GlaMixer(3, 16, 24, 8.0, 4), DenseFF(40, 1.0)),
    layer("parallel", PairMixer(att(4, 2, 16, 24, 0.3, 5.0, 8, 100.0), ssd(2, 12, 10, 1, 1, 4), 0.7, 1.3), DenseFF(24, 2.5)),
    layer("latent_attention", lat(3, 8, 8, 12, 20, 24, 0.2, 50.0, (4.0, 64.0, 4.0, 0.5)), None),
    layer("parallel", PairMixer(att(2, 2, 24, 8, 0.15), ssd(4, 6, 8, 2, 3, 2), 1.0, 0.5), DenseFF(56, 0.75))))
# Q: what P does not have: a latent layer first, with a plain rotation of half of its strip; one kv head for all query
#    heads; a filter of one tap (no convolution state); every head a group of its own; keys wider than values in the gla
#    layer and one head; a latent layer without a rotated strip (the sink alone); scales of one
FIP_Q = FipitarConfig("Fipitar", width=96, vocab=89, norm_eps=1e-6, layers=(
    layer("latent_attention", lat(2, 16, 8, 8, 12, 40, 0.25, 500.0, None, 4), DenseFF(32, 3.0)),
    layer("parallel", PairMixer(att(3, 1, 8, 16, 0.35, 2.0, 8, 1e6), ssd(3, 8, 16, 3, 1, 1), 1.0, 1.0), None),
    layer("gla", GlaMixer(1, 40, 8, 2.0, 3), DenseFF(48, 1.5)),
    layer("latent_attention", lat(5, 8, 0, 16, 24, 16, 0.3), DenseFF(16, 0.5)),
    layer("gla", GlaMixer(4, 8, 8, 32.0, 8), None)))
# R: sizes the tensor-core kernels take: attention heads of 32 x 64, 128 x 16 and 16 x 16, 8 query heads on 2 kv heads
#    (their rows packed into one tile), latent rows of 64 + 16 and of 128 + 32 with 20 heads (more rows a token than a
#    decode tile has), bent frequencies whose bend lies outside the pairs
FIP_R = FipitarConfig("Fipitar", width=128, vocab=301, norm_eps=2e-6, layers=(
    layer("parallel", PairMixer(att(8, 2, 32, 64, 0.2, 10.0, 32, 1e5), ssd(4, 32, 16, 2, 2, 3), 0.9, 1.1), DenseFF(64, 1.5)),
    layer("latent_attention", lat(4, 32, 16, 48, 40, 64, 0.18, 1e4, (2.0, 4096.0, 32.0, 1.0)), DenseFF(96, 2.0)),
    layer("parallel", PairMixer(att(2, 1, 128, 16, 0.09, None, 64, 1e4), ssd(2, 16, 64, 1, 4, 4), 0.5, 2.0), None),
    layer("gla", GlaMixer(2, 64, 32, 16.0, 8), DenseFF(32, 1.0)),
    layer("latent_attention", lat(20, 16, 32, 8, 24, 128, 0.12, 1e5, (8.0, 128.0, 16.0, 2.0)), None),
    layer("parallel", PairMixer(att(4, 4, 16, 16, 0.25, 30.0, 8, 100.0), ssd(1, 8, 8, 1, 1, 2), 1.5, 0.25), DenseFF(48, 4.0))))
# S: recurrent layers only -- the model keeps nothing per position, the cache manager has no group and takes no page
FIP_S = FipitarConfig("Fipitar", width=48, vocab=61, norm_eps=1e-5, layers=(
    layer("gla", GlaMixer(2, 16, 8, 4.0, 2), DenseFF(16, 1.0)),
    layer("gla", GlaMixer(1, 32, 48, 64.0, 5), None)))
# Z: sizes that are multiples of neither 8 nor 16, so that no 16-byte form of any kernel applies, a page of 5 positions
FIP_Z = FipitarConfig("Fipitar", width=100, vocab=53, norm_eps=1e-5, layers=(
    layer("parallel", PairMixer(att(3, 3, 12, 20, 0.3, 4.0, 6, 300.0), ssd(3, 10, 6, 3, 5, 3), 0.8, 0.9), DenseFF(28, 1.25)),
    layer("latent_attention", lat(3, 6, 10, 14, 18, 22, 0.3, 70.0, (3.0, 32.0, 2.0, 0.25), 6), None),
    layer("gla", GlaMixer(2, 20, 12, 6.0, 7), DenseFF(12, 2.0)),
    layer("parallel", PairMixer(att(5, 1, 6, 10, 0.4), ssd(2, 6, 20, 1, 2, 5), 1.2, 0.6), DenseFF(44, 0.9))))
CONFIGS = {"P": (FIP_P, 31, 8), "Q": (FIP_Q, 32, 16), "R": (FIP_R, 33, 16), "S": (FIP_S, 34, 32),
           "Z": (FIP_Z, 35, 5)}       # config, seed, page size

# Readers near 1/sqrt(fan in); the sinks, the decay's bias and the step sizes of order 1 so that they matter; the second
# matrix of the decay's narrow product large, so that decays differ from channel to channel
STD_BY_NAME = ((".sink", 1.5), ("a2.b", 1.0), ("mix.a2", 1.0), ("A_log", 0.5), ("dt_bias", 0.7), ("conv.b", 0.3),
               (".conv", 0.5), ("embed", 0.7))


def random_config(seed):
    """a configuration drawn at random: 2 to 5 layers of any kind in any order, sizes from small sets that include 1, odd
    sizes, multiples of 16 (which the tensor-core kernels take) and keys wider and narrower than values"""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        kind = pick("gla", "latent_attention", "parallel")
        if kind == "gla":
            mixer = GlaMixer(pick(1, 2, 3), pick(8, 16, 24, 40, 64), pick(8, 16, 20, 48), pick(1.0, 4.0, 16.0), pick(2, 4, 16))
        elif kind == "latent_attention":
            rd = pick(0, 4, 8, 16, 32)
            dims = pick(rd, rd // 2 * 2 // 2 * 2) if rd else 0
            dims = dims - dims % 2
            scaling = pick(None, (2.0, 2048.0, 32.0, 1.0), (4.0, 64.0, 4.0, 0.5)) if dims else None
            rank = pick(16, 24, 32, 48, 64)
            mixer = LatentMixer(heads=pick(1, 2, 4, 5, 18), dim=pick(8, 16, 32), vdim=pick(8, 12, 16, 32), q_rank=pick(8, 24, 40),
                                kv_rank=rank, scale=pick(0.1, 0.2, 0.3), rot_dim=rd,
                                rot=Rotation(dims, pick(100.0, 1e4, 2.5e5), scaling) if dims else None)
        else:
            kv = pick(1, 2, 3)
            dim = pick(8, 12, 16, 32, 64)
            rot = pick(0, dim // 2 - (dim // 2) % 2, dim)
            left = AttentionMixer(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=dim, vdim=pick(8, 16, 20, 32, 64), scale=pick(0.1, 0.2, 0.35),
                                  softcap=pick(None, 2.0, 30.0), rot=Rotation(rot, pick(100.0, 5e5)) if rot else None)
            groups = pick(1, 2)
            heads, vdim = groups * pick(1, 2, 3), pick(4, 8, 16)
            parts = pick(1, 2, heads) if (heads * vdim) % 2 == 0 else 1
            right = SsdMixer(heads=heads, vdim=vdim, state=pick(4, 8, 16, 48), groups=groups,
                             norm_groups=parts if (heads * vdim) % parts == 0 else 1, conv=pick(1, 2, 3, 4))
            mixer = PairMixer(left, right, pick(0.6, 1.0), pick(1.1, 0.5))
        layers.append(FipitarLayer(kind, mixer, pick(None, DenseFF(pick(16, 24, 40, 64), pick(0.5, 1.5, 7.0)))))
    return FipitarConfig("Fipitar", width=pick(32, 48, 64, 96, 100), vocab=pick(50, 97, 128), norm_eps=pick(1e-5, 1e-6),
                         layers=tuple(layers))


def make_folder(tmp, name, store="float32"):
    from mashbox_b200.weights.random_init import write_model_folder
    cfg, seed, _ = CONFIGS[name]
    d = os.path.join(str(tmp), f"fip_{name}_{store}")
    if not os.path.isdir(d):
        write_model_folder(d, cfg, seed, dtype=getattr(torch, store), std=cfg.width ** -0.5, norm_std=0.1,
                           std_by_name=STD_BY_NAME)
    return d


@functools.lru_cache(maxsize=None)
def _model(folder):
    return read_model(folder)


@functools.lru_cache(maxsize=64)
def _logits(folder, tokens):
    cfg, W = _model(folder)
    return plain.forward(cfg, W, list(tokens)).numpy()


def plain_logits(folder, tokens):
    """float64 logits (T, V) of the plain implementation for one whole sequence"""
    return _logits(folder, tuple(int(t) for t in tokens))


def prompts_for(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0].vocab, n).tolist() for n in lengths]


def row_nmse(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return ((got - want) ** 2).sum(-1) / np.maximum((want ** 2).sum(-1), 1e-300)


# float32 against the float64 plain model: every product and sum is float32; the bar follows from a measurement: a
# sublayer's output is normed before it joins the stream, so rounding noise is brought back to the stream's own scale in
# every sublayer; the plain model itself multiplies the variance of a small perturbation of its embedding by up to 2,400
# on the way to the logits, and a float32 implementation rounds (6e-8 relative) some dozens of times: 1e-13 x 2,400 x 10
# is 2e-9.
# bfloat16 against the exact model: half of the rows under a twentieth of the bar, nine in ten under the bar (so no more
# than a tenth of the rows over it: the rows after such a one inherit its error through the recurrent states), and the mean
# of all but the worst twentieth under a fifth of it; the worst rows themselves are not bounded.  With random weights a recurrence's output (a sum over the state that is a hundred times a single
# term) cancels at some token to a twentieth of its usual size, and the norm after it brings what is left -- rounding noise
# included -- back to full scale: at such a row two CORRECT bfloat16 implementations (the plain attention kernel and the
# tensor-core one, which differ by an ulp here and there two layers earlier) were measured 0.4 apart in NMSE, each
# matching a float64 scan of its own inputs to 1e-5.  A wrong key, a window one token off or a lost state moves most rows
# after it by order 1, which the median and the tenth-worst row catch; exactness is float32's to show.
BAR = {"float32": 1e-8, "bfloat16": 1e-2}
BAR_SAME = {"float32": 1e-9, "bfloat16": 1e-2}


def assert_close(got, want, dtype, what, bar=None):
    got = np.asarray(got, np.float64)
    assert got.shape == np.asarray(want).shape, (what, got.shape, np.asarray(want).shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    e = row_nmse(got, want)
    limit = (bar or BAR)[dtype]
    if dtype == "float32":
        assert e.max() <= limit, f"{what}: float32 NMSE {e.max():.3e} at row {int(e.argmax())}"
    else:
        over = int((e > limit).sum())
        srt = np.sort(e)
        kept = srt[:len(e) - len(e) // 20] if len(e) >= 20 else srt[:0]
        mean = float(kept.mean()) if len(kept) else 0.0
        p90 = float(srt[(len(e) * 9) // 10]) if len(e) >= 20 else 0.0
        ok = over <= len(e) // 10 and float(np.median(e)) <= limit / 20 and p90 <= limit and mean <= limit / 5
        if len(e) < 20:                     # a few rows: each under the bar
            ok = float(e.max()) <= limit
        assert ok, f"{what}: bfloat16: {over} of {len(e)} rows over {limit:.0e}, worst {e.max():.3e} at row " \
                   f"{int(e.argmax())}, median {np.median(e):.3e}, ninth decile {p90:.3e}, mean without the worst twentieth {mean:.3e}"
    return float(e.max())
