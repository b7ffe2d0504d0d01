"""Small Tosevik configurations with random weights, and the plain implementation's logits for them."""
import functools
import os

import numpy as np
import torch

from mashbox_b200.config.tosevik import ExpertsFF, PairMixer, RetentionMixer, SigmoidMixer, TosevikConfig, TosevikLayer
from tests.plain import tosevik as plain
from tests.plain.llama import read_model


def ret(heads, dim, vdim, decay, rot=0, base=10000.0):
    return RetentionMixer(heads=heads, dim=dim, vdim=vdim, decay=tuple(decay), rot_dims=rot, rot_base=base)


def sig(heads, kv, dim, vdim, scale, temp=None):
    return SigmoidMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale,
                        temp_coef=temp[0] if temp else None, temp_every=temp[1] if temp else None)


def layer(kind, mixer, mlp):
    return TosevikLayer(kind, mixer, mlp)


# T: every size differs from layer to layer where it may.  Retention heads whose keys and values differ in size, a
#    rotation of part of a head and of none of it, decays from 0.5 to 1; attention with two query heads per kv head, a
#    query temperature that moves every 7 positions; experts in 3 groups of which 2 are kept with 3 chosen and a shared
#    expert; ungrouped experts without one; a layer without a feed-forward
TOS_T = TosevikConfig("Tosevik", width=64, vocab=131, norm_eps=1e-5, layers=(
    layer("retention", ret(3, 16, 24, (0.5, 0.9, 0.995), rot=8, base=100.0), ExpertsFF(32, 12, 3, 1.7, 3, 2, 40)),
    layer("parallel", PairMixer(sig(4, 2, 16, 24, 0.2, (0.4, 7)), ret(2, 24, 16, (0.97, 1.0), rot=24, base=5000.0)),
          ExpertsFF(48, 6, 2, 1.0, 1, 1, None)),
    layer("retention", ret(2, 8, 40, (0.75, 0.99)), None),
    layer("parallel", PairMixer(sig(2, 2, 24, 8, 0.1), ret(4, 8, 8, (0.9, 0.95, 0.98, 0.999), rot=4)),
          ExpertsFF(24, 8, 2, 2.5, 4, 1, 16))))
# U: what T does not have: an attention layer first, one kv head for all query heads, one chosen expert, every expert a
#    group of its own, a temperature that moves at every position, one retention head
TOS_U = TosevikConfig("Tosevik", width=96, vocab=89, norm_eps=1e-6, layers=(
    layer("parallel", PairMixer(sig(3, 1, 8, 16, 0.35, (1.0, 1)), ret(1, 40, 24, (0.98,), rot=40, base=1e6)),
          ExpertsFF(24, 6, 1, 1.0, 6, 2, 64)),
    layer("retention", ret(5, 8, 8, (0.6, 0.8, 0.9, 0.95, 0.99), rot=8), ExpertsFF(40, 4, 4, 0.5, 2, 2, None)),
    layer("parallel", PairMixer(sig(6, 3, 16, 8, 0.25), ret(2, 16, 48, (0.93, 0.9995))), None)))
# V: sizes the tensor-core kernels take: attention heads of 64 x 64, 32 x 128 and 128 x 32, 8 query heads on 2 kv heads
#    (their rows packed into one tile), retention heads of 64 x 32
TOS_V = TosevikConfig("Tosevik", width=128, vocab=301, norm_eps=2e-6, layers=(
    layer("parallel", PairMixer(sig(8, 2, 64, 64, 0.12, (0.5, 16)), ret(4, 64, 32, (0.9, 0.99, 0.995, 0.999), rot=64, base=1e5)),
          ExpertsFF(64, 16, 4, 2.0, 4, 2, 96)),
    layer("retention", ret(2, 32, 64, (0.96, 0.999), rot=16), ExpertsFF(32, 4, 2, 1.5, 2, 1, 32)),
    layer("parallel", PairMixer(sig(4, 4, 32, 128, 0.15), ret(2, 16, 16, (0.9, 0.99), rot=16)), None),
    layer("parallel", PairMixer(sig(2, 1, 128, 32, 0.08, (0.3, 50)), ret(1, 128, 16, (0.99,), rot=32)),
          ExpertsFF(128, 4, 1, 1.0, 1, 1, None))))
# W: retention layers only -- the model keeps nothing per position, the cache manager has no group and takes no page
TOS_W = TosevikConfig("Tosevik", width=48, vocab=61, norm_eps=1e-5, layers=(
    layer("retention", ret(2, 16, 8, (0.9, 0.99), rot=16, base=50.0), ExpertsFF(16, 4, 2, 1.2, 2, 2, 8)),
    layer("retention", ret(1, 32, 48, (0.97,), rot=2), None)))
# Z: sizes that are multiples of neither 8 nor 16, so that no 16-byte form of any kernel applies, a page of 5 positions,
#    attention layers only but for one
TOS_Z = TosevikConfig("Tosevik", width=100, vocab=53, norm_eps=1e-5, layers=(
    layer("parallel", PairMixer(sig(3, 3, 12, 20, 0.3, (0.7, 3)), ret(3, 10, 6, (0.8, 0.9, 0.99), rot=6)),
          ExpertsFF(28, 6, 2, 0.9, 3, 2, 12)),
    layer("parallel", PairMixer(sig(5, 1, 6, 10, 0.4), ret(2, 12, 20, (0.95, 0.5), rot=12, base=300.0)), None),
    layer("retention", ret(2, 20, 12, (0.99, 0.9)), ExpertsFF(12, 5, 3, 2.0, 1, 1, 44))))
CONFIGS = {"T": (TOS_T, 21, 8), "U": (TOS_U, 22, 16), "V": (TOS_V, 23, 16), "W": (TOS_W, 24, 32),
           "Z": (TOS_Z, 25, 5)}       # config, seed, page size

# Readers near 1/sqrt(fan in), writers into the stream small; the router wide enough that the chosen experts are seldom
# a close call; the biases of the attention heads of order 1 so that they matter.
STD_BY_NAME = ((".pb", 1.0), ("mlp.router", 0.6), (".sg", 0.3), ("mix.o", 0.1), ("left.o", 0.2), ("right.o", 0.2),
               (".down", 0.1), ("embed", 0.7))


def make_folder(tmp, name, store="float32"):
    from mashbox_b200.weights.random_init import write_model_folder
    cfg, seed, _ = CONFIGS[name]
    d = os.path.join(str(tmp), f"tos_{name}_{store}")
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


# float32 against the float64 plain model: every product and sum is float32.  bfloat16 against the exact model: a row
# may reach the bar, a twentieth of the rows ten times the bar (a token whose last chosen expert is a close call gets
# another expert than the exact model gives it), and the mean over the rows a fifth of the bar.
BAR = {"float32": 1e-9, "bfloat16": 1e-2}
BAR_SAME = {"float32": 1e-10, "bfloat16": 1e-2}


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
        mean = float(e.mean()) if len(e) >= 20 else 0.0
        assert over <= len(e) // 20 and e.max() <= 10 * limit and mean <= (limit / 5 if bar is None else limit / 10), \
            f"{what}: bfloat16: {over} of {len(e)} rows over {limit:.0e}, worst {e.max():.3e} at row {int(e.argmax())}, " \
            f"mean {e.mean():.3e}"
    return float(e.max())
