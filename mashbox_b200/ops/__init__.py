"""Python faces of the hand-written CUDA kernels (mashbox_b200/csrc) and of the one library routine the engine uses.

Every function works on CUDA tensors, launches on torch's current stream and raises KernelError when the kernel
refuses the sizes.  There is no CPU or library fallback for a kernel: if the extension cannot be built or no GPU is
there, the call fails.  The only library call is the bf16 matrix product (cuBLAS through torch.mm), which stands where
the reference engine, too, hands its contractions to a library (src/mashbox/ops/dense16.py:73-75).
"""
import ctypes

import torch

from ..errors import KernelError
from .build import load_library

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

# bf16 products accumulate in float32 all the way: no reduced-precision reduction inside the library
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False

DEVICE_ERRORS = {1: "a token id outside the vocabulary", 2: "a position whose cache page the block table does not hold",
                 3: "a page id outside the cache pool", 4: "a bounded wait inside a kernel ran out",
                 5: "a position outside the learned position table"}


def _suffix(dtype):
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"no kernel for dtype {dtype}")


def _p(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    # the current stream's handle; torch.cuda.current_stream() costs several microseconds a call, a tenth of the host's
    # time in a step of two hundred launches, the raw accessor next to nothing
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("mashbox_b200 kernels run on CUDA tensors only; there is no CPU fallback")


COUNTERS = {"launches": 0}      # launches of this package's own kernels (a graph replay adds what it captured)


def _check(code, what):
    if code == 0:
        COUNTERS["launches"] += 1
        return
    if code == -2:
        raise KernelError(f"{what}: the kernel does not take these sizes")
    if code == -6:
        raise KernelError(f"{what}: the driver refused a tensor map")
    raise KernelError(f"{what}: CUDA error {code} at launch")


# Scratch that the faces below keep per device (partial sums, counters, reduction buffers) is made once and grows
# when a larger problem comes.  A captured graph holds the addresses it was captured with, so whoever replays graphs
# must capture again after a growth: scratch_generation() changes whenever any such buffer was replaced.
_scratch = {"generation": 0}


def scratch_generation():
    return _scratch["generation"]


# Programmatic dependent launch along the chain of kernels of a small step: a kernel of these libraries may start while
# the kernel before it in the stream still runs, sets itself up (the weight-streaming products send for their first
# weights), and waits for that kernel by itself before it touches anything a kernel writes.  One switch per library,
# set through set_pdl(); the engine's option "pdl" turns it on.
PDL = {"on": False}
_PDL_SETTERS = {"gemm_stream": "mb_gemm_stream_set_pdl", "elementwise": "mb_elementwise_set_pdl",
                "attention_tma": "mb_attn_tma_set_pdl"}
_pdl_applied = {}


def _apply_pdl(lib):
    name = _PDL_SETTERS.get(lib)
    if name is not None and _pdl_applied.get(lib) != PDL["on"]:
        f = getattr(load_library(lib), name, None)
        if f is not None:
            f.argtypes = [c_int]
            f(1 if PDL["on"] else 0)
        _pdl_applied[lib] = PDL["on"]


def set_pdl(on):
    PDL["on"] = bool(on)
    for lib in list(_pdl_applied):
        _apply_pdl(lib)


_fn_cache = {}


def _fn(lib, name, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        _pdl_applied.setdefault(lib, None)
        _apply_pdl(lib)
        f = getattr(load_library(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    return f


def new_error_word(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


_error_words = {}


def error_word(device):
    """The one error word per device that kernels without a caller-supplied word report to (the engine's step function
    uses it for all its kernels, so one read after a step sees every report)."""
    key = str(torch.device(device))
    if key not in _error_words:
        _error_words[key] = new_error_word(device)
    return _error_words[key]


def check_error_word(err):
    """Reads the device error word (a synchronisation) and raises if a kernel left a code there."""
    code = int(err.item())
    if code:
        err.zero_()
        raise KernelError("a kernel reported: " + DEVICE_ERRORS.get(code, f"code {code}"))


# ------------------------------------------------------------------------------------------------ elementwise
def embed(tokens, table, x, err, scale=1.0):
    """x[n] = table[tokens[n]] * scale into the float32 residual stream x (N, D)."""
    _cuda(tokens, table, x)
    N, D = x.shape
    f = _fn("elementwise", "mb_embed_" + _suffix(table.dtype),
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(f(_p(tokens), _p(table), _p(x), N, D, table.shape[0], float(scale), _p(err), _stream()), "embed")


def add_rmsnorm(x, delta, delta_bias, weight, eps, out, rows=None):
    """v = x (+ delta (+ delta_bias)); written back to x unless rows is given; out = v * rsqrt(mean(v^2)+eps) * weight.
    x (N, D) float32; delta (N, D) and out in the activation dtype; weight, delta_bias float32; rows int32 indexes."""
    _cuda(x, delta, weight, out, rows)
    D = x.shape[1]
    n_out = out.shape[0]
    f = _fn("elementwise", "mb_add_rmsnorm_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(delta_bias), _p(rows), _p(weight), float(eps), _p(out), n_out, D, _stream()),
           "add_rmsnorm")


def add_rmsnorm_pair(x, delta1, delta2, weight1, weight2, eps, out1, out2=None, rows=None):
    """v = x (+ delta1) (+ delta2), written back to x unless rows is given; out1 = v * rsqrt(mean(v^2) + eps) * weight1
    and, with weight2, out2 = the same with weight2 (one pass, one sum of squares).  x (N, D) float32; deltas and outs in
    the activation dtype; weights float32; rows int32 indexes."""
    _cuda(x, delta1, delta2, weight1, weight2, out1, out2, rows)
    D = x.shape[1]
    f = _fn("elementwise", "mb_add_rmsnorm_pair_" + _suffix(out1.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
             c_void_p])
    _check(f(_p(x), _p(delta1), _p(delta2), _p(rows), _p(weight1), _p(weight2), float(eps), _p(out1), _p(out2),
             out1.shape[0], D, _stream()), "add_rmsnorm_pair")


def add_rmsnorm_pair_conv(x, delta1, delta2, weight1, weight2, eps, out1, out2, conv_w, state, slots):
    """add_rmsnorm_pair for a step in which every sequence brings one token, with the short causal convolution of the
    first output folded in: out1 <- out1 + conv(out1) over the row's state.  conv_w (taps, D) float32 tap by tap, state
    (slots, (taps - 1) D) float32 (a view; replaced by the step's), slots int32 (N,) the state slot of every row.  D a
    multiple of 8, taps at least 2; the same bits as add_rmsnorm_pair followed by short_conv(residual=True)."""
    _cuda(x, delta1, delta2, weight1, weight2, out1, out2, conv_w, state, slots)
    D = x.shape[1]
    if conv_w.shape[1] != D or not conv_w.is_contiguous():
        raise KernelError("add_rmsnorm_pair_conv: the filters must be a contiguous (taps, width) tensor")
    f = _fn("elementwise", "mb_add_rmsnorm_pair_conv_" + _suffix(out1.dtype),
            [c_void_p] * 5 + [c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p,
                              c_int, c_void_p])
    _check(f(_p(x), _p(delta1), _p(delta2), _p(weight1), _p(weight2), float(eps), _p(out1), _p(out2), out1.shape[0], D,
             _p(conv_w), _p(state), state.stride(0), _p(slots), conv_w.shape[0], _stream()), "add_rmsnorm_pair_conv")


def xielu(z, out, ap, an):
    """out = ap z^2 + z/2 where z > 0, an (exp(z) - 1 - z) + z/2 elsewhere; z and out (N, F) in the activation dtype"""
    _cuda(z, out)
    f = _fn("elementwise", "mb_xielu_" + _suffix(out.dtype),
            [c_void_p, c_void_p, ctypes.c_longlong, c_float, c_float, c_void_p])
    _check(f(_p(z), _p(out), z.numel(), float(ap), float(an), _stream()), "xielu")


# ------------------------------------------------------------------------------------------------ short convolutions
def short_conv(x, w, state, seq, out, residual=False):
    """out = (x if residual) + causal_conv(x): x, out (N, C) in the activation dtype, w (taps, C) float32, one filter per
    channel, held tap by tap (the transpose of how checkpoints store them).  state (slots, taps - 1, C) float32 (a view: rows C apart, slots state.stride(0) apart) holds every
    sequence's last taps - 1 inputs and is replaced by this step's.  seq = (tok_seq, q_start, q_len, state_slot) int32
    device arrays: per token its sequence's index in the step; per sequence its first token, length and state slot."""
    _cuda(x, w, state, out, *seq)
    N, C = x.shape
    taps = w.shape[0]
    if w.shape[1] != C or not w.is_contiguous():
        raise KernelError("short_conv: the filters must be a contiguous (taps, channels) tensor")
    f = _fn("short_conv", "mb_short_conv_" + _suffix(x.dtype),
            [c_void_p, c_void_p, c_void_p, ctypes.c_longlong] + [c_void_p] * 5 + [c_int] * 5 + [c_void_p])
    _check(f(_p(x), _p(w), _p(state), state.stride(0) if state is not None else 0, *[_p(t) for t in seq], _p(out), N,
             seq[1].shape[0], C, taps, 1 if residual else 0, _stream()), "short_conv")


def conv_rope_kv_write(qkv, bias, w, state, seq, positions, tok_row, table, q_out, kpool, vpool, freqs, QU, KU, VH, dim,
                       vdim, kper, RD, page, num_pages, err):
    """What follows a fused q/k/v product whose outputs pass a short convolution: rows of qkv (N, (QU + KU) dim + VH
    vdim) = [query units | key units | value heads] get their bias, are convolved over time per channel (w (C, taps)
    float32 or None; state and seq as short_conv), the first RD dims of every query and key unit are rotated by the
    token's position (dim i with dim i + RD/2; freqs (RD/2,) float32 or None), queries go to q_out (N, QU dim), keys
    and values into the pages of the token's position: kpool (pages, VH, page, kper dim) takes `kper` key units per kv
    head, vpool (pages, VH, page, vdim).  KU = VH = 0: the rows hold queries only."""
    _cuda(qkv, bias, w, state, positions, tok_row, table, q_out, kpool, vpool, freqs, *seq)
    N = qkv.shape[0]
    taps = 1 if w is None else w.shape[0]
    if w is not None and (w.shape[1] != qkv.shape[1] or not w.is_contiguous()):
        raise KernelError("conv_rope_kv_write: the filters must be a contiguous (taps, channels) tensor")
    f = _fn("short_conv", "mb_conv_rope_kv_write_" + _suffix(qkv.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_longlong] + [c_void_p] * 7 + [c_int] + [c_void_p] * 4
            + [c_int] * 12 + [c_void_p, c_void_p])
    _check(f(_p(qkv), _p(bias), _p(w), _p(state), state.stride(0) if state is not None else 0, *[_p(t) for t in seq],
             _p(positions), _p(tok_row), _p(table), table.shape[1] if table is not None else 0, _p(q_out), _p(kpool),
             _p(vpool), _p(freqs), N, seq[1].shape[0], QU, KU, VH, dim, vdim, kper, RD, page, num_pages, taps, _p(err),
             _stream()),
           "conv_rope_kv_write")


def rope_kv_write(qkv, bias, positions, tok_seq, table, kpool, vpool, freqs, H, KV, HD, RD, pairing, page, num_pages,
                  err):
    """qkv (N, (H + 2 KV) HD): adds bias, rotates q in place, writes rotated k and v to their pages (kpool/vpool None:
    q only).  freqs (RD/2,) float32 angle per position step, None = no rotation; pairing 0 adjacent, 1 halves."""
    _cuda(qkv, positions, tok_seq, table, kpool, vpool, freqs)
    N = qkv.shape[0]
    f = _fn("elementwise", "mb_rope_kv_write_" + _suffix(qkv.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 8
            + [c_void_p, c_void_p])
    _check(f(_p(qkv), _p(bias), _p(positions), _p(tok_seq), _p(table), table.shape[1], _p(kpool), _p(vpool), _p(freqs),
             N, H, KV, HD, RD, pairing, page, num_pages, _p(err), _stream()), "rope_kv_write")


def patch_tokens(dst, src, pairs, n):
    """dst[pairs[2i]] = src[pairs[2i+1]] for i < n (int32 tensors on the device)"""
    _cuda(dst, src, pairs)
    f = _fn("elementwise", "mb_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(dst), _p(src), _p(pairs), int(n), _stream()), "patch_tokens")


def swiglu(gu, out):
    """gu (N, 2F) = [gate | up] -> out (N, F) = silu(gate) * up"""
    _cuda(gu, out)
    N, F = out.shape
    f = _fn("elementwise", "mb_swiglu_" + _suffix(out.dtype), [c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(gu), _p(out), N, F, _stream()), "swiglu")


# ------------------------------------------------------------------------------------------------ row-wise kernels
c_ll = ctypes.c_longlong


def embed_positions(tokens, positions, table, pos_table, x, err, scale=1.0):
    """x[n] = table[tokens[n]] * scale + pos_table[positions[n]] into the float32 residual stream x (N, D)"""
    _cuda(tokens, positions, table, pos_table, x)
    N, D = x.shape
    f = _fn("rowwise", "mb_embed_pos_" + _suffix(table.dtype),
            [c_void_p] * 5 + [c_int] * 4 + [c_float, c_void_p, c_void_p])
    _check(f(_p(tokens), _p(positions), _p(table), _p(pos_table), _p(x), N, D, table.shape[0], pos_table.shape[0],
             float(scale), _p(err), _stream()), "embed_positions")


def post_norm_add(x, delta, post_w, post_eps, next_w=None, next_eps=0.0, normed=None, copy=None):
    """x (N, D) float32 += delta / sqrt(mean(delta^2) + post_eps) * post_w (delta in the activation dtype, post_w float32);
    with next_w and normed: normed = x / sqrt(mean(x^2) + next_eps) * next_w; copy: x in the activation dtype"""
    _cuda(x, delta, post_w, next_w, normed, copy)
    N, D = x.shape
    f = _fn("rowwise", "mb_post_norm_add_" + _suffix(delta.dtype),
            [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(post_w), float(post_eps), _p(next_w), float(next_eps), _p(normed), _p(copy), N, D,
             _stream()), "post_norm_add")


def rms_segments(rows, off_a, w_a, out_a, off_b, w_b, pool, positions, tok_row, table, page, num_pages, eps, err):
    """Two stretches of columns of rows (N, C), each divided by its root mean square and multiplied by a weight of its
    own: columns off_a .. off_a + len(w_a) go to out_a (N, len(w_a)); columns off_b .. off_b + len(w_b) go into pool
    (pages, 1, page, len(w_b)) at the page and slot of the token's position (w_b None: no second stretch)."""
    _cuda(rows, w_a, out_a, w_b, pool, positions, tok_row, table)
    N, C = rows.shape
    wa = 0 if w_a is None else w_a.shape[0]
    wb = 0 if w_b is None else w_b.shape[0]
    f = _fn("rowwise", "mb_rms_segments_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_p(rows), rows.stride(0), off_a, wa, _p(w_a), _p(out_a), off_b, wb, _p(w_b), _p(pool), _p(positions),
             _p(tok_row), _p(table), table.shape[1] if table is not None else 0, page, num_pages, float(eps), N, _p(err),
             _stream()), "rms_segments")


def rms_segments_wide(rows, off_a, w_a, out_a, off_b, w_b, pool, positions, tok_row, table, page, num_pages, eps, err):
    """rms_segments whose second stretch goes into the first len(w_b) values of a cache row that is wider than it: pool
    (pages, 1, page, row)"""
    _cuda(rows, w_a, out_a, w_b, pool, positions, tok_row, table)
    N = rows.shape[0]
    wa = 0 if w_a is None else w_a.shape[0]
    wb = 0 if w_b is None else w_b.shape[0]
    f = _fn("rowwise", "mb_rms_segments_wide_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(f(_p(rows), rows.stride(0), off_a, wa, _p(w_a), _p(out_a), off_b, wb, _p(w_b), _p(pool),
             pool.shape[-1] if pool is not None else 0, _p(positions), _p(tok_row), _p(table),
             table.shape[1] if table is not None else 0, page, num_pages, float(eps), N, _p(err), _stream()),
           "rms_segments_wide")


def gated_gather(z, tokens, table, off, out, err):
    """out[n, j] = gelu_tanh(z[n, j]) * table[tokens[n], off + j]; z, out (N, W), table (V, any) in the activation dtype"""
    _cuda(z, tokens, table, out)
    N, W = z.shape
    f = _fn("rowwise", "mb_gated_gather_" + _suffix(z.dtype),
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(z), _p(tokens), _p(table), table.stride(0), int(off), _p(out), N, W, table.shape[0], _p(err), _stream()),
           "gated_gather")


def sigmoid_mul(o, gate):
    """o (N, C) *= sigmoid(gate), in place; gate a view (N, C) whose rows may be further apart than C"""
    _cuda(o, gate)
    N, C = o.shape
    if gate.stride(1) != 1:
        raise KernelError("sigmoid_mul: the gate's columns must be contiguous")
    f = _fn("rowwise", "mb_sigmoid_mul_" + _suffix(o.dtype), [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(o), _p(gate), gate.stride(0), N, C, _stream()), "sigmoid_mul")


# The per-head products run on the package's plain kernel up to this many tokens (and always in float32); larger bf16
# steps hand them to the library's batched product.
HEAD_PRODUCT = {"tokens": 32}


def head_product_strided(x, I, w, out, J, heads, transposed):
    """head_product on stretches of wider heads: x (N, heads * in_head) of whose every head the first I values are read,
    out (N, heads * out_head) of whose every head the first J values are written; w as in head_product."""
    _cuda(x, w, out)
    N = x.shape[0]
    in_head, out_head = x.shape[1] // heads, out.shape[1] // heads
    if tuple(w.shape) != ((heads * I, J) if transposed else (heads * J, I)) or not w.is_contiguous():
        raise KernelError("head_product: the matrix does not fit the heads")
    if x.dtype == torch.bfloat16 and N > HEAD_PRODUCT["tokens"]:
        a = x.view(N, heads, in_head)[:, :, :I].transpose(0, 1)
        b = w.view(heads, I, J) if transposed else w.view(heads, J, I).transpose(1, 2)
        out.view(N, heads, out_head)[:, :, :J].copy_(torch.bmm(a, b).transpose(0, 1))
        return out
    sh, si, sj = (I * J, J, 1) if transposed else (I * J, 1, I)
    f = _fn("rowwise", "mb_head_product_strided_" + _suffix(x.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_void_p])
    _check(f(_p(x), in_head, _p(w), _p(out), out_head, N, heads, I, J, sh, si, sj, _stream()), "head_product")
    return out


def head_product(x, w, out, heads, transposed):
    """A projection applied head by head.  x (N, heads * I), out (N, heads * J), w the stored matrix:
    transposed=False: w (heads * J, I) and out[n, h] = w[h] x[n, h] (rows of a head side by side);
    transposed=True:  w (heads * I, J) and out[n, h] = w[h]^T x[n, h] (the same matrix applied from the other side)."""
    _cuda(x, w, out)
    N = x.shape[0]
    I, J = x.shape[1] // heads, out.shape[1] // heads
    if tuple(w.shape) != ((heads * I, J) if transposed else (heads * J, I)) or not w.is_contiguous():
        raise KernelError("head_product: the matrix does not fit the heads")
    if x.dtype == torch.bfloat16 and N > HEAD_PRODUCT["tokens"]:
        a = x.view(N, heads, I).transpose(0, 1)
        b = w.view(heads, I, J) if transposed else w.view(heads, J, I).transpose(1, 2)
        out.view(N, heads, J).copy_(torch.bmm(a, b).transpose(0, 1))
        return out
    sh, si, sj = (I * J, J, 1) if transposed else (I * J, 1, I)
    f = _fn("rowwise", "mb_head_product_" + _suffix(x.dtype),
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_void_p])
    _check(f(_p(x), _p(w), _p(out), N, heads, I, J, sh, si, sj, _stream()), "head_product")
    return out


def scale_rows(y, s):
    """y (float32) *= s, in place"""
    _cuda(y)
    f = _fn("rowwise", "mb_scale_rows", [c_void_p, c_float, c_ll, c_void_p])
    _check(f(_p(y), float(s), y.numel(), _stream()), "scale_rows")


# ------------------------------------------------------------------------------------------------ gated delta rule
def delta_gates(qkv, low, wide, A_log, dt_bias, q, k, v, g, beta, H, G, dim, vdim, unit_eps=1e-6):
    """What the delta rule reads, in float32, from a layer's products.  qkv (N, 2 G dim + H vdim) = [q | k | v] (after
    their convolutions): silu; q, k to unit vectors per head, x / sqrt(sum x^2 + unit_eps), q also times dim^-1/2.
    low (N, >= H): beta = sigmoid of its first H columns.  wide (N, H dim + H vdim): g = exp(-exp(A_log[h])
    softplus(wide[:, :H dim] + dt_bias)).  Outputs q, k (N, G dim), v (N, H vdim), g (N, H dim), beta (N, H)."""
    _cuda(qkv, low, wide, A_log, dt_bias, q, k, v, g, beta)
    f = _fn("delta_rule", "mb_delta_gates_" + _suffix(qkv.dtype),
            [c_void_p, c_void_p, c_int] + [c_void_p] * 8 + [c_int] * 5 + [c_float, c_void_p])
    _check(f(_p(qkv), _p(low), low.stride(0), _p(wide), _p(A_log), _p(dt_bias), _p(q), _p(k), _p(v), _p(g), _p(beta),
             qkv.shape[0], H, G, dim, vdim, float(unit_eps), _stream()), "delta_gates")


def delta_rule(q, k, v, g, beta, o, state, seq, H, G, dim, vdim):
    """Per sequence and head, token by token: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k (N, G dim), v, o (N, H vdim), g (N, H dim), beta (N, H), all float32; state (slots, H dim vdim) float32 (a view,
    slots state.stride(0) apart), read at the start of each sequence's stretch and replaced at its end.
    seq = (q_start, q_len, state_slot) int32 device arrays, one entry per sequence of the step."""
    _cuda(q, k, v, g, beta, o, state, *seq)
    f = _fn("delta_rule", "mb_delta_rule", [c_void_p] * 7 + [c_ll] + [c_void_p] * 3 + [c_int] * 5 + [c_void_p])
    _check(f(_p(q), _p(k), _p(v), _p(g), _p(beta), _p(o), _p(state), state.stride(0), _p(seq[0]), _p(seq[1]), _p(seq[2]),
             seq[0].shape[0], H, G, dim, vdim, _stream()), "delta_rule")


def delta_rule_lanes(lanes):
    """how many threads hold a column of the state: 0 = the default (8, with as many values each as the keys need),
    16 or 32 = that many (fewer values a thread, more shuffles); a measuring switch"""
    f = getattr(load_library("delta_rule"), "mb_delta_rule_set_lanes")
    f.argtypes = [c_int]
    f(int(lanes))


def gated_rms(o, gate, w, out, H, vdim, eps, silu=False):
    """out[n, h] = o[n, h] / sqrt(mean(o[n, h]^2) + eps) * w * sigmoid(gate[n, h]) per head; o (N, H vdim) float32, gate
    (N, H vdim) of the activation dtype whose rows may be further apart, w (vdim,) float32 or None (no weight), out the
    activation dtype; silu: the gate is silu(gate) instead of sigmoid(gate)"""
    _cuda(o, gate, w, out)
    f = _fn("delta_rule", "mb_gated_rms_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_p(o), _p(gate), gate.stride(0), 0, _p(w), _p(out), o.shape[0], H, vdim, float(eps), int(bool(silu)), _stream()),
           "gated_rms")


# ------------------------------------------------------------------------------------------------ the stream of blocks with Dynamic Tanh
def dyt(x, delta, alpha, w, b, out, rows=None, delta2=None):
    """x (N, D) float32 += delta (+ delta2) (in place unless rows picks rows); out = tanh(alpha x) * w + b.  out is of
    the activation dtype (that of delta when given) or float32 -- it may be x itself"""
    _cuda(x, delta, delta2, w, b, out, rows)
    D = x.shape[1]
    n_out = x.shape[0] if rows is None else rows.shape[0]
    act = delta.dtype if delta is not None else out.dtype
    out_float = out.dtype == torch.float32 and act != torch.float32
    f = _fn("stream", "mb_dyt_" + _suffix(act),
            [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(delta2), float(alpha), _p(w), _p(b), _p(out), int(out_float), _p(rows), n_out, D, _stream()),
           "dyt")


def depth_average(x, delta, hist, coef, idx, normed=None, next_norm=None):
    """y = x + delta;  hist[idx + 1] = y;  x = sum_(j <= idx + 1) coef[j] hist[j].  x (N, D) float32, delta (N, D) of the
    activation dtype or None, hist (slots, rows >= N, D) float32, coef (idx + 2,) float32.  With normed and
    next_norm = (alpha, w, b): normed = tanh(alpha x) * w + b, of the activation dtype."""
    _cuda(x, delta, hist, coef, normed)
    N, D = x.shape
    act = delta.dtype if delta is not None else (normed.dtype if normed is not None else torch.float32)
    if coef.numel() < idx + 2 or hist.shape[0] < idx + 2 or hist.shape[1] < N:
        raise KernelError("depth_average: the history or the coefficients are too short")
    na, nw, nb = next_norm if normed is not None else (0.0, None, None)
    f = _fn("stream", "mb_depth_average_" + _suffix(act),
            [c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(delta), _p(hist), hist.stride(0), _p(coef), int(idx), float(na), _p(nw), _p(nb), _p(normed), N, D,
             _stream()), "depth_average")


def rms_pair_mean(a, b, wa, wb, out, eps):
    """out = (a / rms(a) * wa + b / rms(b) * wb) / 2 row by row; a, b, out (N, D) of the activation dtype, wa, wb float32"""
    _cuda(a, b, wa, wb, out)
    N, D = a.shape
    f = _fn("stream", "mb_rms_pair_mean_" + _suffix(a.dtype), [c_void_p] * 5 + [c_int, c_int, c_float, c_void_p])
    _check(f(_p(a), _p(b), _p(wa), _p(wb), _p(out), N, D, float(eps), _stream()), "rms_pair_mean")


# ------------------------------------------------------------------------------------------------ retention
def retention_prep(rows, q_off, k_off, v_off, positions, freqs, q, k, v, H, dim, vdim, rotary_dim, k_scale):
    """rows (N, C) of the activation dtype holds q at column q_off, k at k_off (H dim each) and v at v_off (H vdim); the
    first rotary_dim values of every head of q and k turn by position * freqs[i] (value i with value i + rotary_dim / 2);
    k is multiplied by k_scale after that; q, k (N, H, dim) and v (N, H, vdim) float32"""
    _cuda(rows, positions, freqs, q, k, v)
    f = _fn("retention", "mb_retention_prep_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p] + [c_int] * 5
            + [c_float, c_void_p])
    _check(f(_p(rows), rows.stride(0), int(q_off), int(k_off), int(v_off), _p(positions), _p(freqs), _p(q), _p(k), _p(v),
             rows.shape[0], H, dim, vdim, int(rotary_dim), float(k_scale), _stream()), "retention_prep")


# Steps with more than `chunk_tokens` tokens a sequence run the split form of the recurrence, in segments of
# `segment_tokens` -- when the scan would leave the device short of blocks (fewer than `scan_blocks`): the split form walks
# every token twice, which pays only while the scan's blocks do not fill the multiprocessors.
RETENTION = {"chunk_tokens": 64, "segment_tokens": 128, "scan_blocks": 148}


def retention_scan_blocks(S, H, vdim):
    """blocks of the scan form: a block takes 16 columns of one head's state of one sequence"""
    return S * H * (-(-vdim // 16))


def retention_splits(N, S, H, vdim):
    """whether a step of N tokens in S sequences runs the split form"""
    return N > RETENTION["chunk_tokens"] * S and retention_scan_blocks(S, H, vdim) < RETENTION["scan_blocks"]


def retention_carry_rows(N, S, segment=None):
    """rows of the carry buffer that the split form wants for N tokens in S sequences"""
    return N // int(segment or RETENTION["segment_tokens"]) + S


def retention(q, k, v, decay, o, state, seq, H, dim, vdim, chunked=False, segment=None, carry=None):
    """Per sequence and head, token by token: S <- decay[h] S + k v^T; o = S^T q.  q, k (N, H, dim), v, o (N, H, vdim)
    float32; decay (H,) float32; state (slots, >= H vdim dim) float32, a head's state stored (vdim, dim);
    seq = (q_start, q_len, state_slot) device arrays.  chunked: the split form, which cuts every sequence into segments of
    `segment` tokens that run side by side; carry (>= retention_carry_rows(N, S, segment), H vdim dim) float32 is its
    scratch (made here when absent)."""
    _cuda(q, k, v, decay, o, state, *seq)
    if not chunked:
        f = _fn("retention", "mb_retention_scan", [c_void_p] * 6 + [c_ll] + [c_void_p] * 3 + [c_int] * 4 + [c_void_p])
        _check(f(_p(q), _p(k), _p(v), _p(decay), _p(o), _p(state), state.stride(0), _p(seq[0]), _p(seq[1]), _p(seq[2]),
                 seq[0].numel(), H, dim, vdim, _stream()), "retention")
        return
    import torch
    N, S = q.shape[0], seq[0].numel()
    segment = int(segment or RETENTION["segment_tokens"])
    if carry is None:
        carry = torch.empty(retention_carry_rows(N, S, segment), H * vdim * dim, dtype=torch.float32, device=q.device)
    _cuda(carry)
    f = _fn("retention", "mb_retention_split",
            [c_void_p] * 6 + [c_ll] + [c_void_p] * 3 + [c_int] * 6 + [c_void_p, c_int, c_void_p])
    _check(f(_p(q), _p(k), _p(v), _p(decay), _p(o), _p(state), state.stride(0), _p(seq[0]), _p(seq[1]), _p(seq[2]), S, N, H,
             dim, vdim, segment, _p(carry), carry.shape[0], _stream()), "retention")
    COUNTERS["launches"] += 2           # the first pass, the carry, the second pass


# ------------------------------------------------------------------------------------------------ attention with sigmoid weights
def sigmoid_attention_prep(rows, qw, kw, positions, tok_row, table, q_out, kpool, vpool, H, G, dim, vdim, page, num_pages,
                           eps, temp_coef, temp_every, err):
    """rows (N, H dim + G dim + G vdim) = [q | k | v]: q and k divided by the root mean square of their whole row and
    multiplied by qw, kw (float32, a value per channel), q also by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1)
    (temp_every 0: no such factor); every head's v divided by its own root mean square.  q goes to q_out (N, H dim), k and
    v into kpool (pages, G, page, dim) and vpool (pages, G, page, vdim) at the token's position (None: not written)."""
    _cuda(rows, qw, kw, positions, tok_row, table, q_out, kpool, vpool)
    f = _fn("attention_sigmoid", "mb_sigattn_prep_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
            + [c_int] * 7 + [c_float, c_float, c_int, c_void_p, c_void_p])
    _check(f(_p(rows), rows.stride(0), _p(qw), _p(kw), _p(positions), _p(tok_row), _p(table), table.shape[1], _p(q_out),
             _p(kpool), _p(vpool), rows.shape[0], H, G, dim, vdim, page, num_pages, float(eps), float(temp_coef),
             int(temp_every), _p(err), _stream()), "sigmoid_attention_prep")


def sigmoid_attention_simple(q, out, positions, tok_row, table, kpool, vpool, slopes, bias, H, G, dim, vdim, page, num_pages,
                             scale, err):
    """out[n, h] = sum over the keys j <= p of sigmoid(scale q[n, h] . k_j - slopes[h] (p - j) + bias[h]) v_j, one warp per
    (token, head), keys in ascending position; slopes, bias (H,) float32 or None"""
    _cuda(q, out, positions, tok_row, table, kpool, vpool, slopes, bias)
    f = _fn("attention_sigmoid", "mb_sigattn_simple_" + _suffix(q.dtype),
            [c_void_p] * 5 + [c_int] + [c_void_p] * 4 + [c_int] * 7 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(positions), _p(tok_row), _p(table), table.shape[1], _p(kpool), _p(vpool), _p(slopes),
             _p(bias), q.shape[0], H, G, dim, vdim, page, num_pages, float(scale), _p(err), _stream()),
           "sigmoid_attention_simple")


SIGMOID_MMA_ROWS, SIGMOID_DECODE_ROWS, SIGMOID_MAX_SPLITS = 64, 16, 16


def sigmoid_attention_mma_supports(dim, vdim):
    """the tensor-core kernel of the attention with sigmoid weights takes these head sizes (bfloat16 only)"""
    return dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128


def _sigmoid_mma_library(dim, vdim):
    from .build import variant
    return variant(f"attention_sigmoid_mma_{dim}_{vdim}", "attention_sigmoid_mma.cu", [f"-DSIG_DIM={dim}", f"-DSIG_VD={vdim}"])


def sigmoid_attention_mma(q, out, items, n_items, q_start, q_len, pos0, seq_row, table, kpool, vpool, slopes, bias, H, G, dim,
                          vdim, page, num_pages, scale, err):
    """Attention with sigmoid weights on tensor cores (bfloat16): the same result as sigmoid_attention_simple.  items:
    n_items (sequence, tile of 64 packed rows) pairs; q_start, q_len, pos0, seq_row per sequence.  The kernel is compiled
    for the pair (dim, vdim) the first time it is asked for."""
    _cuda(q, out, items, q_start, q_len, pos0, seq_row, table, kpool, vpool, slopes, bias)
    if q.dtype != torch.bfloat16 or not sigmoid_attention_mma_supports(dim, vdim):
        raise KernelError(f"sigmoid_attention_mma: no kernel for {q.dtype} with head sizes {dim} and {vdim}")
    f = _fn(_sigmoid_mma_library(dim, vdim), "mb_sigattn_mma", [c_void_p] * 5 + [c_int] + [c_void_p] * 5 + [c_int]
            + [c_void_p] * 2 + [c_int] * 4 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(kpool), _p(vpool), _p(items), int(n_items), _p(q_start), _p(q_len), _p(pos0), _p(seq_row),
             _p(table), table.shape[1], _p(slopes), _p(bias), H, G, page, num_pages, float(scale), _p(err), _stream()),
           "sigmoid_attention_mma")


def sigmoid_attention_mma_decode(q, out, items, n_items, slots, n_slots, part_o, q_start, q_len, pos0, seq_row, table, kpool,
                                 vpool, slopes, bias, H, G, dim, vdim, page, num_pages, scale, err):
    """The decode form of sigmoid_attention_mma, for sequences of at most 16 packed rows: items are n_items (sequence,
    split, number of splits, slot) quadruples, the keys of a sequence cut into splits that run side by side; slots:
    n_slots (sequence, number of splits) pairs of the sequences that are cut, whose partial sums a second kernel adds in
    the order of the splits from part_o (n_slots * G * 16 * 16, vdim) float32."""
    _cuda(q, out, items, slots, part_o, q_start, q_len, pos0, seq_row, table, kpool, vpool, slopes, bias)
    if q.dtype != torch.bfloat16 or not sigmoid_attention_mma_supports(dim, vdim):
        raise KernelError(f"sigmoid_attention_mma_decode: no kernel for {q.dtype} with head sizes {dim} and {vdim}")
    f = _fn(_sigmoid_mma_library(dim, vdim), "mb_sigattn_mma_decode", [c_void_p] * 5 + [c_int, c_void_p, c_int]
            + [c_void_p] * 6 + [c_int] + [c_void_p] * 2 + [c_int] * 4 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(kpool), _p(vpool), _p(items), int(n_items), _p(slots), int(n_slots), _p(part_o),
             _p(q_start), _p(q_len), _p(pos0), _p(seq_row), _p(table), table.shape[1], _p(slopes), _p(bias), H, G, page,
             num_pages, float(scale), _p(err), _stream()), "sigmoid_attention_mma_decode")
    if n_slots:
        COUNTERS["launches"] += 1


def sigmoid_attention_tc5_supports(dim, vdim, page):
    """the tcgen05 kernel's form with sigmoid weights: keys and values of one width, 64 or 128"""
    return dim == vdim and attention_tc5_supports(dim, page)


def sigmoid_attention_tc5_rows():
    """packed query rows of one work item of the tcgen05 kernel (two query tiles of 128 rows share the K and V tiles)"""
    return 256


def sigmoid_attention_tc5(q, out, items, n_items, q_start, q_len, pos0, seq_row, table, kpool, vpool, slopes, bias, H, G, dim,
                          vdim, page, num_pages, scale, err):
    """The prompt form of the attention with sigmoid weights on tcgen05 (the result of sigmoid_attention_simple): items
    are n_items (sequence, tile of 256 packed rows, 0, 1) quadruples, heaviest first."""
    _cuda(q, out, items, q_start, q_len, pos0, seq_row, table, kpool, vpool, slopes, bias)
    if q.dtype != torch.bfloat16 or not sigmoid_attention_tc5_supports(dim, vdim, page):
        raise KernelError(f"sigmoid_attention_tc5: no kernel for {q.dtype}, head sizes {dim} and {vdim}, pages of {page}")
    f = _fn("attention_tc5_sig", "mb_attn_tc5_sig_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int] + [c_int] * 6 + [c_float] + [c_void_p] * 4)
    _check(f(_p(q), H * dim, _p(out), _p(kpool), _p(vpool), _p(items), int(n_items), _p(q_start), _p(q_len), _p(pos0),
             _p(seq_row), _p(table), table.shape[1], H, G, dim, page, num_pages, 0, float(scale), _p(slopes), _p(bias),
             _p(err), _stream()), "sigmoid_attention_tc5")


# ------------------------------------------------------------------------------------------------ routed experts
def moe_select(z, correction, ids, wts, groups=1, keep=1, experts=None, softmax=False, worth="top2", scale=1.0):
    """z (N, >= E) float32 router logits (E = experts, default: every column) -> ids (N, top) int32, wts (N, top) float32:
    scores sigmoid(z), or softmax(z) over the E experts; chosen by score + correction among the experts of the `keep` best
    of `groups` runs of neighbours (a run's worth: the sum of its two largest, "top2", or its largest, "max"); the
    weights are the chosen experts' scores times `scale`"""
    _cuda(z, correction, ids, wts)
    N = z.shape[0]
    E = int(experts) if experts is not None else z.shape[1]
    if worth not in ("top2", "max"):
        raise KernelError(f"moe_select: a group's worth is top2 or max, not {worth!r}")
    f = _fn("moe", "mb_moe_select", [c_void_p, c_int] + [c_void_p] * 3 + [c_int] * 7 + [c_float, c_void_p])
    _check(f(_p(z), z.stride(0), _p(correction), _p(ids), _p(wts), N, E, ids.shape[1], int(groups), int(keep),
             int(bool(softmax)), int(worth == "max"), float(scale), _stream()), "moe_select")


def _expert_views(wg, wu, wd):
    D = wg.shape[2]
    if (wg.stride(1), wg.stride(2)) != (D, 1) or wu.stride() != wg.stride() or not wd.is_contiguous():
        raise KernelError("the experts' matrices must have contiguous rows, gate and up alike")


def moe_experts(h, ids, wg, wu, wd, y, limit, alpha, act=None, shift=1.0):
    """y[n, k] = Wd[e] (g sigmoid(alpha g) (u + shift)), g = min(Wg[e] h[n], limit), u = clamp(Wu[e] h[n], -limit, limit),
    e = ids[n, k].  h (N, D); wg, wu (E, F, D), whole tensors or the two halves of one (E, 2F, D) tensor; wd (E, D, F);
    y (N, top, D) float32; act (N * top, F) float32: working memory (made here when not given)"""
    _cuda(h, ids, wg, wu, wd, y, act)
    N, D = h.shape
    E, F, _ = wg.shape
    _expert_views(wg, wu, wd)
    if act is None:
        act = torch.empty((N * ids.shape[1], F), dtype=torch.float32, device=h.device)
    f = _fn("moe", "mb_moe_experts_" + _suffix(h.dtype),
            [c_void_p] * 4 + [c_ll] + [c_void_p] * 3 + [c_int] * 5 + [c_float, c_float, c_float, c_void_p])
    _check(f(_p(h), _p(ids), _p(wg), _p(wu), wg.stride(0), _p(wd), _p(y), _p(act), N, D, F, E, ids.shape[1], float(limit),
             float(alpha), float(shift), _stream()), "moe_experts")
    COUNTERS["launches"] += 1


# Steps of more tokens than this run the experts on tensor-core tiles over the pairs sorted by expert (bf16 only).
MOE_GROUPED = {"tokens": 16}


def moe_grouped_supports(N, D, F, dtype):
    return dtype == torch.bfloat16 and N > MOE_GROUPED["tokens"] and D % 8 == 0 and F % 8 == 0


def moe_grouped_scratch(N, top, E):
    """-> the number of int32 values moe_grouped needs as scratch"""
    P = N * top
    return P + (E + 1) + 3 * (P // 64 + E) + 1 + 3


def moe_grouped(h, ids, wg, wu, wd, y, act, scratch, limit, alpha, shift=1.0):
    """moe_experts for steps of many tokens, bf16: the (token, place) pairs are sorted by expert on the device and every
    expert's rows run through tensor-core tiles.  act (N * top, F) bf16 and scratch (moe_grouped_scratch values, int32)
    are working memory."""
    _cuda(h, ids, wg, wu, wd, y, act, scratch)
    N, D = h.shape
    E, F, _ = wg.shape
    top = ids.shape[1]
    P = N * top
    max_tiles = P // 64 + E
    if scratch.numel() < moe_grouped_scratch(N, top, E) or scratch.dtype != torch.int32:
        raise KernelError("moe_grouped: the scratch is too small")
    sorted_, offsets = scratch[:P], scratch[P:P + E + 1]
    tiles = scratch[P + E + 1:P + E + 1 + 3 * max_tiles]
    n_tiles = scratch[P + E + 1 + 3 * max_tiles:]
    _expert_views(wg, wu, wd)
    f = _fn("moe", "mb_moe_grouped_bf16", [c_void_p] * 4 + [c_ll] + [c_void_p] * 7 + [c_int] * 5 + [c_float, c_float, c_float, c_void_p])
    _check(f(_p(h), _p(ids), _p(wg), _p(wu), wg.stride(0), _p(wd), _p(y), _p(act), _p(sorted_), _p(offsets), _p(tiles),
             _p(n_tiles), N, D, F, E, top, float(limit), float(alpha), float(shift), _stream()), "moe_grouped")
    COUNTERS["launches"] += 2


def moe_tc5_supports(N, D, F, dtype):
    """steps of 128 tokens and more: the experts' products run on the tcgen05 product in its grouped form"""
    return dtype == torch.bfloat16 and N >= 128 and D % 8 == 0 and F % 8 == 0 and TC5["experts"]


def moe_tc5_tiles(N, top, E):
    """-> the number of tiles of 128 rows the sorted layout has room for (every expert's rows start at a multiple of 128)"""
    return N * top // 128 + E


def moe_tc5(h, ids, wts, wgu, wd, out, rows, act, y, scratch, limit, alpha, shift=1.0, shared=None, gate=None):
    """The routed experts of a step of many tokens, bf16: ids (N, top) and wts from moe_select; wgu (E, 2F, D), every
    expert's gate rows then its up rows; wd (E, D, F); out (N, D).  Working memory, with T = moe_tc5_tiles(N, top, E):
    rows (128 T, D) bf16, act (128 T, F) bf16, y (128 T, D) float32, scratch (N top + T) int32.  shared (N, D) and gate
    (float32, one logit per token, rows gate.stride(0) apart): see moe_combine."""
    _cuda(h, ids, wts, wgu, wd, out, rows, act, y, scratch, shared, gate)
    N, D = h.shape
    E, F = wgu.shape[0], wgu.shape[1] // 2
    top = ids.shape[1]
    T = moe_tc5_tiles(N, top, E)
    if rows.shape[0] < 128 * T or act.shape[0] < 128 * T or y.shape[0] < 128 * T or scratch.numel() < N * top + T:
        raise KernelError("moe_tc5: the working memory is too small")
    place, tile_expert = scratch[:N * top], scratch[N * top:N * top + T]
    f = _fn("moe", "mb_moe_sort_gather", [c_void_p] * 5 + [c_int] * 4 + [c_void_p])
    _check(f(_p(h), _p(ids), _p(place), _p(tile_expert), _p(rows), N, D, E, top, _stream()), "moe_sort_gather")
    err = error_word(h.device)
    f = _fn("gemm_tc5", "mb_gemm_tc5_grouped_gated_bf16",
            [c_void_p] * 3 + [c_int] * 3 + [c_void_p, c_int, c_float, c_float, c_float, c_void_p, c_void_p])
    _check(f(_p(rows), _p(wgu), _p(act), 128 * T, F, D, _p(tile_expert), E, float(limit), float(alpha), float(shift), _p(err),
             _stream()),
           "gemm_tc5_grouped_gated")
    f = _fn("gemm_tc5", "mb_gemm_tc5_grouped_f32out", [c_void_p] * 3 + [c_int] * 3 + [c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(act), _p(wd), _p(y), 128 * T, D, F, _p(tile_expert), E, _p(err), _stream()), "gemm_tc5_grouped")
    f = _fn("moe", "mb_moe_combine_rows", [c_void_p] * 4 + [c_int] * 3 + [c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(y), _p(place), _p(wts), _p(out), N, D, top, _p(shared), _p(gate), gate.stride(0) if gate is not None else 0,
             _stream()), "moe_combine_rows")
    COUNTERS["launches"] += 1


def moe_combine(y, wts, out, shared=None, gate=None):
    """out[n] = sum_k wts[n, k] y[n, k] (places in order); y (N, top, D) float32, out (N, D) the activation dtype.
    shared (N, D) of the activation dtype: the output of an expert every token uses, added times sigmoid(gate[n]) (gate:
    float32, one logit per token, rows gate.stride(0) apart; None: added as it is)"""
    _cuda(y, wts, out, shared, gate)
    N, top, D = y.shape
    f = _fn("moe", "mb_moe_combine_" + _suffix(out.dtype), [c_void_p] * 3 + [c_int] * 3 + [c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(y), _p(wts), _p(out), N, D, top, _p(shared), _p(gate), gate.stride(0) if gate is not None else 0, _stream()),
           "moe_combine")


def linear(a, w, out=None, out_dtype=None):
    """a (N, K) @ w (M, K)^T -> (N, M).  float32: the package's own fixed-order FFMA kernel (no TF32, no tensor
    cores).  bfloat16: cuBLAS with float accumulation; out_dtype float32 keeps the accumulator's precision."""
    _cuda(a, w)
    N, K = a.shape
    M = w.shape[0]
    if a.dtype == torch.float32:
        if out is None:
            out = torch.empty((N, M), dtype=torch.float32, device=a.device)
        f = _fn("gemm_f32", "mb_gemm_f32", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(f(_p(a), _p(w), _p(out), N, M, K, _stream()), "gemm_f32")
        return out
    if tc5_supports(N, M, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want in (torch.bfloat16, torch.float32):
            return linear_tc5(a, w, out, "plain" if want == torch.bfloat16 else "float")
    if gemv_supports(N, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want == torch.bfloat16:      # the output head stays with the library
            return linear_gemv(a, w, out, "plain")
    if stream_supports(N, K) and a.is_contiguous() and w.is_contiguous() and a.dtype == torch.bfloat16 and M % 8 == 0:
        want = a.dtype if out_dtype is None else out_dtype
        if out is None:
            out = torch.empty((N, M), dtype=want, device=a.device)
        if out.is_contiguous() and out.dtype == want and want in (torch.bfloat16, torch.float32):
            return linear_stream(a, w, out, "plain" if want == torch.bfloat16 else "float")
    if out_dtype is not None and out_dtype != a.dtype:
        r = torch.mm(a, w.t(), out_dtype=out_dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is not None:
        return torch.mm(a, w.t(), out=out)
    return torch.mm(a, w.t())


# The package's own tcgen05 product for prompt portions (128 tokens or more).  "swiglu": the fused gate/up product
# (measured 317 us against 310 + 33 us for the library product and the separate gate kernel at 2,048 tokens of the
# Llama-3.1-8B shape); "plain": every product (87 to 97 % of the library's speed, so off by default).
TC5 = {"swiglu": True, "plain": False, "experts": True}


def tc5_supports(N, M, K, mode="plain"):
    return TC5["swiglu" if mode == "swiglu" else "plain"] and N >= 128 and K >= 8 and K % 8 == 0 and M % 8 == 0


def linear_tc5(a, w, out, mode="plain"):
    """a (N, K) bf16, w (M, K) bf16 (mode "swiglu": (2M, K) = [gate rows | up rows]) -> out (N, M): bf16 for "plain" and
    "swiglu" (silu(gate) * up), float32 for "float".  TMA + tcgen05.mma with the accumulator in tensor memory."""
    _cuda(a, w, out)
    N, K = a.shape
    name = {"plain": "mb_gemm_tc5_bf16", "swiglu": "mb_gemm_tc5_swiglu_bf16", "float": "mb_gemm_tc5_f32out"}[mode]
    f = _fn("gemm_tc5", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(a), _p(w), _p(out), N, out.shape[1], K, _p(error_word(a.device)), _stream()), "gemm_tc5")
    return out


# Matrix-vector products (one warp per two rows of W, or a block per two long rows; no tensor core): the kernels take up
# to 4 tokens, the engine uses them where they beat the library, which is at ONE token.  Measured inside captured
# graphs on the Llama-3.1-8B shapes at one token, own / library: output product 10.8 / 13.0 us, QKV 12.2 / 11.7, down
# 21.2 / 24.9, fused gate/up + SwiGLU 39.0 / 39.2 + 2.3; at two tokens the arithmetic (bf16 to float conversions on
# the FMA pipe) already costs more than the stream.  GEMV[mode] = the most tokens the engine gives the kernel (0: never);
# "fused": the forms that normalise the residual stream themselves or add their product into it (see small_fused_supports).
# A limit of -1 leaves the choice to the width of the product's input (GEMV_AUTO: the matrix-vector kernels up to that
# many tokens below that width, else the weight-streaming products).  One request, 128 new tokens after 32 of prompt,
# through Engine.admit/step (python bench.py --workload 1b-single and the like), matrix-vector / streaming: Llama-3.2-1B
# shape (width 2,048) 1,378 / 987 tokens/s, Llama-3.2-3B shape (3,072) 605 / 498, Falcon3-1B shape (2,048) 1,047 / 765,
# Llama-3.1-8B shape (4,096) 328 / 315 (the same at 8,192 tokens of context: 3.35 ms a step either way): the advantage
# shrinks with the width (+40 %, +21 %, +4 %), so the line for one token is drawn between 4,096 and 5,120.  At two
# tokens (2,048 of context) the 1B shape takes 0.88 / 0.91 ms a step, the 3B shape 1.98 / 1.88, the 8B shape 3.84 /
# 3.55; at three they are level, at four the streaming products win everywhere.
GEMV = {"swiglu": 1, "plain": 1, "fused": 1}
GEMV_AUTO = ((2560, 2), (4608, 1))            # (narrower than, tokens), the first line that applies


def _gemv_limit(mode, K):
    v = GEMV[mode]
    if v >= 0:
        return v
    if not PDL["on"]:
        return 1
    for width, tokens in GEMV_AUTO:
        if K < width:
            return tokens
    return 0


def gemv_supports(N, K, mode="plain"):
    return 1 <= N <= min(4, _gemv_limit("swiglu" if mode == "swiglu" else "plain", K)) and K >= 8 and K % 8 == 0


def linear_gemv_normed(x, norm_w, eps, w, out, mode="plain"):
    """x (N <= 4, K) float32 residual stream, norm_w (K) float32 -> out (N, M) bf16 = rmsnorm(x) W^T ("swiglu": W is
    (2M, K) and out = silu(gate) * up), the normalised row rounded to bf16 as the norm kernel would store it."""
    _cuda(x, norm_w, w, out)
    N, K = x.shape
    name = {"plain": "mb_gemv_normed_bf16", "swiglu": "mb_gemv_normed_swiglu_bf16"}[mode]
    f = _fn("gemv", name, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(norm_w), float(eps), _p(w), _p(out), N, out.shape[1], K, _stream()), "gemv_normed")
    return out


def linear_gemv_normed_qkv(x, norm_w, eps, w, out, bias, positions, tok_seq, table, kpool, vpool, freqs, H, KV, HD, RD,
                           pairing, page, num_pages, err):
    """x (N <= 4, K) float32 residual stream -> the fused q/k/v product of rmsnorm(x) with the rotate-and-store step in
    its epilogue: out (N, (H + 2 KV) HD) bf16 receives the rotated q heads, the rotated k and the v heads go into the
    pages of the tokens' positions (kpool None: dropped), as rope_kv_write would leave them."""
    _cuda(x, norm_w, w, out, bias, positions, tok_seq, table, kpool, vpool, freqs)
    N, K = x.shape
    f = _fn("gemv", "mb_gemv_normed_qkv_bf16",
            [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_void_p])
    _check(f(_p(x), _p(norm_w), float(eps), _p(w), _p(out), N, out.shape[1], K, _p(bias), _p(positions), _p(tok_seq),
             _p(table), table.shape[1], _p(kpool), _p(vpool), _p(freqs), H, KV, HD, RD, pairing, page, num_pages,
             _p(err), _stream()), "gemv_normed_qkv")
    return out


def linear_gemv_residual(a, w, x, bias=None):
    """x (N <= 4, M) float32 += a (N, K) bf16 @ w (M, K)^T (+ bias (M) float32), in place"""
    _cuda(a, w, x, bias)
    N, K = a.shape
    f = _fn("gemv", "mb_gemv_residual", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(a), _p(w), _p(x), _p(bias), N, x.shape[1], K, _stream()), "gemv_residual")
    return x


def linear_gemv(a, w, out, mode="plain"):
    """a (N <= 4, K) bf16, w (M, K) bf16 ("swiglu": (2M, K)) -> out (N, M): bf16, or float32 for mode "float"."""
    _cuda(a, w, out)
    N, K = a.shape
    name = {"plain": "mb_gemv_bf16", "swiglu": "mb_gemv_swiglu_bf16", "float": "mb_gemv_f32out"}[mode]
    f = _fn("gemv", name, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(a), _p(w), _p(out), N, out.shape[1], K, _stream()), "gemv")
    return out


# The weight-streaming products for steps of 2 to 16 tokens (gemm_stream.cu): W is cut into row tiles low enough that
# most SMs get one (no tile shared for the layer's own matrices), streamed by TMA, mma.sync on the tiles.  The product
# that ends a sublayer adds into the residual stream and leaves what the norm after it needs (sums of squares, rows
# times the norm's weight); the product after that norm runs on those rows and scales its sums by 1 / rms; gate/up has
# SwiGLU in its epilogue.  A layer is then six kernels instead of ten.  Measured inside captured graphs on the
# Llama-3.1-8B shapes at 8 tokens, own / library, us: output product with the residual add 11.4 / 12.0 (+ the add in the
# norm kernel), q/k/v of the normalised stream 12.0 / 11.9 + norm 3.8, gate/up with SwiGLU 40.6 / 40.2 + norm 3.8 + gate
# 2.3, down with the residual add 26.5 / 23.3; the whole decode step at batch 8 (the output head too): 1,720 tokens/s
# against 1,608 with the library's products.  STREAM["tokens"]: the most tokens the engine gives them (0: never).
STREAM = {"tokens": 16}


def configure(options):
    """Engine options that choose between this package's kernels, applied process-wide (the kernels' faces are module
    functions).  pdl (default on): programmatic dependent launch along the chain of kernels of a small step; with it
    the weight-streaming products take steps of one token too when the model is wide enough (GEMV_AUTO)
    (narrower models stay with the matrix-vector kernels, which are launched plainly: launched that way themselves
    they lost 0.7 ms a step on the 8B shape).
    gemv_tokens / stream_tokens: the most tokens of a step the matrix-vector / weight-streaming products take (0: never;
    gemv_tokens unset: by the width)."""
    pdl = bool(options.get("pdl", True))
    set_pdl(pdl)
    for k in GEMV:
        GEMV[k] = int(options["gemv_tokens"]) if "gemv_tokens" in options else (-1 if pdl else 1)
    STREAM["tokens"] = int(options.get("stream_tokens", 16))


_stream_scratch = {}


def stream_supports(N, K):
    return 1 <= N <= min(16, STREAM["tokens"]) and K >= 8 and K % 8 == 0


def _stream_buffers(device, M):
    """(workspace, counters) of the streaming products on this device: the partial sums of row tiles that blocks
    share, and a counter per row tile, zero between launches"""
    lib = load_library("gemm_stream")
    lib.mb_gemm_stream_workspace.restype = ctypes.c_longlong
    key = str(device)
    sc = _stream_scratch.get(key)
    tiles = (M + 31) // 32
    if sc is None or sc[1].numel() < tiles:
        sc = (torch.empty(lib.mb_gemm_stream_workspace(), dtype=torch.float32, device=device),
              torch.zeros(max(tiles, 8192), dtype=torch.int32, device=device))
        _stream_scratch[key] = sc
        _scratch["generation"] += 1
    return sc


def linear_stream(a, w, out, mode="plain", sums=None, eps=0.0):
    """a (N <= 16, K) bf16, w (M, K) bf16 ("swiglu": (2M, K)) -> out (N, M): bf16, or float32 for mode "float".
    sums (ceil(K / 32), 16) float32, if given: a holds rows of a residual stream times a norm's weight and sums the sums
    of squares of those rows by 32 columns, as linear_stream_residual leaves them; out is then the product of
    rmsnorm(x; weight, eps): 1 / rms scales the float sums of the product."""
    _cuda(a, w, out, sums)
    N, K = a.shape
    M = out.shape[1]
    ws, cnt = _stream_buffers(a.device, M)
    f = _fn("gemm_stream", "mb_gemm_stream", [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(a), _p(sums), float(eps), _p(w), _p(out), N, M, K, {"plain": 0, "swiglu": 1, "float": 2}[mode], _p(ws),
             _p(cnt), _p(error_word(a.device)), _stream()), "gemm_stream")
    return out


def linear_stream_residual(a, w, x, bias=None, sums=None, next_w=None, scaled=None):
    """x (N <= 16, M) float32 += a (N, K) bf16 @ w (M, K)^T (+ bias (M) float32), in place.  What the norm that reads x
    next needs, on request: sums (ceil(M / 32), 16) float32 receives the sums of squares of the new rows by 32 columns,
    scaled (N, M) bf16 the new rows times that norm's weight next_w (M) float32."""
    _cuda(a, w, x, bias, sums, next_w, scaled)
    N, K = a.shape
    M = x.shape[1]
    ws, cnt = _stream_buffers(a.device, M)
    f = _fn("gemm_stream", "mb_gemm_stream_residual", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(a), _p(w), _p(x), _p(bias), N, M, K, _p(sums), _p(next_w), _p(scaled), _p(ws), _p(cnt),
             _p(error_word(a.device)), _stream()), "gemm_stream_residual")
    return x


# ---- what the parts call at few tokens: the matrix-vector kernels where they are enabled, else the streaming products.
# "held" is what the product that last added into the residual stream left for the norm after it (sums of squares by 32
# columns, rows times the norm's weight in bf16): the streaming products need it, the matrix-vector kernels read x.
def _use_gemv_fused(N, K):
    return 1 <= N <= min(4, _gemv_limit("fused", K)) and K % 8 == 0 and 8 <= K < 8192 and N * K * 2 <= 48 * 1024


def small_fused_supports(N, K, dtype):
    """True when a step of N tokens of width K can run its layers on the folded kernels: the product that follows a
    norm is the product of the normalised stream without a norm kernel (linear_small_normed), the product that ends a
    sublayer adds into the stream (linear_small_residual)."""
    return dtype == torch.bfloat16 and (_use_gemv_fused(N, K) or stream_supports(N, K))


def small_normed_needs_held(N, K):
    return not _use_gemv_fused(N, K)


def small_qkv_supports(N, K):
    """True when linear_small_normed_qkv takes this step (else: linear_small_normed, then rope_kv_write)"""
    return _use_gemv_fused(N, K)


def linear_small_normed(x, norm_w, eps, w, out, mode="plain", held=None):
    if _use_gemv_fused(*x.shape):
        return linear_gemv_normed(x, norm_w, eps, w, out, mode)
    sums, scaled = held
    return linear_stream(scaled, w, out, mode, sums, eps)


def linear_small_normed_qkv(x, norm_w, eps, w, out, *args):
    return linear_gemv_normed_qkv(x, norm_w, eps, w, out, *args)


def linear_small_residual(a, w, x, bias=None, sums=None, next_w=None, scaled=None):
    """-> True when sums and scaled were filled (see linear_stream_residual)"""
    if _use_gemv_fused(a.shape[0], x.shape[1]) and a.shape[1] % 8 == 0:
        linear_gemv_residual(a, w, x, bias)
        return False
    linear_stream_residual(a, w, x, bias, sums, next_w, scaled)
    return sums is not None and scaled is not None


def fused_swiglu_supports(N, F, K):
    return gemv_supports(N, K, "swiglu") or stream_supports(N, K) or tc5_supports(N, F, K, "swiglu")


def fused_xielu_supports(N, F, K):
    """the up product of a prompt portion with the xIELU activation in its epilogue (the tcgen05 product)"""
    return tc5_supports(N, F, K, "swiglu")


def linear_xielu(a, w, out, ap, an):
    """a (N, K) bf16, w (F, K) bf16 -> out (N, F) bf16 = xielu(a W^T), one kernel; shapes fused_xielu_supports() takes"""
    _cuda(a, w, out)
    N, K = a.shape
    if not (fused_xielu_supports(N, out.shape[1], K) and a.dtype == torch.bfloat16 and a.is_contiguous()
            and w.is_contiguous() and out.is_contiguous()):
        raise KernelError("linear_xielu: no fused kernel takes these sizes")
    f = _fn("gemm_tc5", "mb_gemm_tc5_xielu_bf16", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                                   c_void_p, c_void_p])
    _check(f(_p(a), _p(w), _p(out), N, out.shape[1], K, float(ap), float(an), _p(error_word(a.device)), _stream()),
           "gemm_tc5_xielu")
    return out


def linear_glu_clamped(a, wgu, out, limit, alpha=1.702, shift=1.0):
    """a (N, K) bf16, wgu (2F, K) = [gate rows | up rows] -> out (N, F) = g sigmoid(alpha g) (u + shift) with the clamps of
    glu_clamped, one kernel (the tcgen05 product with the gate in its epilogue); shapes fused_xielu_supports() takes"""
    _cuda(a, wgu, out)
    N, K = a.shape
    if not (tc5_supports(N, out.shape[1], K, "swiglu") and a.dtype == torch.bfloat16 and a.is_contiguous()
            and wgu.is_contiguous() and out.is_contiguous()):
        raise KernelError("linear_glu_clamped: no fused kernel takes these sizes")
    f = _fn("gemm_tc5", "mb_gemm_tc5_glu_clamped_bf16", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                                                         c_float, c_void_p, c_void_p])
    _check(f(_p(a), _p(wgu), _p(out), N, out.shape[1], K, float(limit or 0.0), float(alpha), float(shift),
             _p(error_word(a.device)), _stream()), "gemm_tc5_glu_clamped")
    return out


def linear_swiglu(a, wgu, out):
    """a (N, K) bf16, wgu (2F, K) = [gate rows | up rows] -> out (N, F) = silu(a Wg^T) * (a Wu^T), one kernel: the
    tcgen05 product for prompt portions, the matrix-vector or the weight-streaming kernel for decode batches (where enabled).
    Only for shapes fused_swiglu_supports() takes."""
    _cuda(a, wgu, out)
    N, K = a.shape
    if tc5_supports(N, out.shape[1], K, "swiglu"):
        return linear_tc5(a, wgu, out, "swiglu")
    if gemv_supports(N, K, "swiglu"):
        return linear_gemv(a, wgu, out, "swiglu")
    if stream_supports(N, K):
        return linear_stream(a, wgu, out, "swiglu")
    raise KernelError("linear_swiglu: no fused kernel takes these sizes")


# ------------------------------------------------------------------------------------------------ attention
def attention_simple(q, q_stride, out, positions, tok_seq, table, kpool, vpool, H, KV, HD, page, num_pages, window,
                     scale, err):
    _cuda(q, out, positions, tok_seq, table, kpool, vpool)
    N = out.shape[0]
    f = _fn("attention_simple", "mb_attn_simple_" + _suffix(out.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7
            + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(positions), _p(tok_seq), _p(table), table.shape[1], _p(kpool), _p(vpool), N,
             H, KV, HD, page, num_pages, window or 0, float(scale), _p(err), _stream()), "attention_simple")


def attention_diff_simple(q, out, positions, tok_row, table, kpool, vpool, H, G, dim, vdim, page, num_pages, chunk,
                          scale, lam, gain, eps, err):
    """Differential attention, plain kernel: q (N, H * 2 dim) holds two maps per head, kpool (pages, G, page, 2 dim),
    vpool (pages, G, page, vdim) -> out (N, H vdim) = rmsnorm_head(a_0 - lam a_1) * gain, a_m the softmax attention of
    map m over the keys of the query's own block of `chunk` positions (0: all) up to its position."""
    _cuda(q, out, positions, tok_row, table, kpool, vpool)
    f = _fn("attention_diff", "mb_attn_diff_simple_" + _suffix(q.dtype),
            [c_void_p] * 5 + [c_int, c_void_p, c_void_p] + [c_int] * 8 + [c_float] * 4 + [c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(positions), _p(tok_row), _p(table), table.shape[1], _p(kpool), _p(vpool), q.shape[0], H,
             G, dim, vdim, page, num_pages, int(chunk or 0), float(scale), float(lam), float(gain), float(eps), _p(err),
             _stream()), "attention_diff_simple")


DIFF_MMA_ROWS = 64


def attention_diff_mma_supports(dim, vdim):
    """the tensor-core kernel of the differential attention takes these head sizes (bfloat16 only)"""
    return dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128


def attention_diff_mma_rows():
    """packed query rows (tokens times the query heads of a kv head) of one work item"""
    return DIFF_MMA_ROWS


DIFF_DECODE_ROWS, DIFF_MAX_SPLITS = 16, 16


def attention_diff_mma_decode(q, out, items, n_items, slots, n_slots, part_o, part_ml, q_start, q_len, pos0, seq_row, table,
                              kpool, vpool, H, G, dim, vdim, page, num_pages, chunk, scale, lam, gain, eps, err):
    """The decode form of attention_diff_mma, for sequences of at most 16 packed rows: items are n_items (sequence,
    split, number of splits, slot) quadruples, the keys of a sequence cut into splits that run side by side; slots:
    n_slots (sequence, number of splits) pairs of the sequences that are cut, whose splits a second kernel merges from
    part_o (n_slots * G * 16 * 2 * 16, vdim) and part_ml (the same rows, 2), float32."""
    _cuda(q, out, items, slots, part_o, part_ml, q_start, q_len, pos0, seq_row, table, kpool, vpool)
    if q.dtype != torch.bfloat16 or not attention_diff_mma_supports(dim, vdim):
        raise KernelError(f"attention_diff_mma_decode: no kernel for {q.dtype} with head sizes {dim} and {vdim}")
    from .build import variant
    lib = variant(f"attention_diff_mma_{dim}_{vdim}", "attention_diff_mma.cu", [f"-DDIFF_DIM={dim}", f"-DDIFF_VD={vdim}"])
    f = _fn(lib, "mb_attn_diff_mma_decode", [c_void_p] * 5 + [c_int, c_void_p, c_int] + [c_void_p] * 7 + [c_int] * 6
            + [c_float] * 4 + [c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(kpool), _p(vpool), _p(items), int(n_items), _p(slots), int(n_slots), _p(part_o),
             _p(part_ml), _p(q_start), _p(q_len), _p(pos0), _p(seq_row), _p(table), table.shape[1], H, G, page, num_pages,
             int(chunk or 0), float(scale), float(lam), float(gain), float(eps), _p(err), _stream()),
           "attention_diff_mma_decode")
    if n_slots:
        COUNTERS["launches"] += 1


def attention_diff_mma(q, out, items, n_items, q_start, q_len, pos0, seq_row, table, kpool, vpool, H, G, dim, vdim, page,
                       num_pages, chunk, scale, lam, gain, eps, err):
    """Differential attention on tensor cores (bfloat16): the same result as attention_diff_simple.  items: n_items
    (sequence, tile of 64 packed rows) pairs; q_start, q_len, pos0, seq_row per sequence.  The kernel is compiled for
    the pair (dim, vdim) the first time it is asked for."""
    _cuda(q, out, items, q_start, q_len, pos0, seq_row, table, kpool, vpool)
    if q.dtype != torch.bfloat16 or not attention_diff_mma_supports(dim, vdim):
        raise KernelError(f"attention_diff_mma: no kernel for {q.dtype} with head sizes {dim} and {vdim}")
    from .build import variant
    lib = variant(f"attention_diff_mma_{dim}_{vdim}", "attention_diff_mma.cu", [f"-DDIFF_DIM={dim}", f"-DDIFF_VD={vdim}"])
    f = _fn(lib, "mb_attn_diff_mma", [c_void_p] * 5 + [c_int] + [c_void_p] * 5 + [c_int] * 6 + [c_float] * 4
            + [c_void_p, c_void_p])
    _check(f(_p(q), _p(out), _p(kpool), _p(vpool), _p(items), int(n_items), _p(q_start), _p(q_len), _p(pos0), _p(seq_row),
             _p(table), table.shape[1], H, G, page, num_pages, int(chunk or 0), float(scale), float(lam), float(gain),
             float(eps), _p(err), _stream()), "attention_diff_mma")


def attention_mma_supports(HD):
    """head sizes in steps of 16 up to 256 (16, 32, 64, 128 in one library, the others in a second one)"""
    return 16 <= HD <= 256 and HD % 16 == 0


def _mma_library(HD):
    return "attention_mma" if HD in (16, 32, 64, 128) else "attention_mma_wide"


def attention_mma(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                  table,
                  part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale, err):
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, part_base, table, part_o, part_ml)
    f = _fn(_mma_library(HD), "mb_attn_mma_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, 1 if decode else 0, _p(q_start),
             _p(q_len), _p(pos0), _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml), max_splits, H, KV,
             HD, page, num_pages, window or 0, float(scale), _p(err), _stream()), "attention_mma")


def attention_tma_supports(HD, page):
    return HD in (64, 128) and page in (8, 16, 32, 64)


_merge_counters = {}
MERGE_COUNTERS = 1 << 16


def attention_tma_merges(n_items, KV):
    """True when attention_tma can merge the splits of its items itself (it has a counter for every group)"""
    return n_items * KV <= MERGE_COUNTERS


def attention_tma_folds_rotation(G):
    """True when attention_tma can take the rotate-and-store step of a step of one-token sequences in (rope=...)"""
    return 1 <= G <= 16


_max_cluster = {}


def attention_tma_max_cluster(HD):
    """the most splits of a sequence whose blocks attention_tma can launch as one thread-block cluster (1: none)"""
    if HD not in _max_cluster:
        lib = load_library("attention_tma")
        lib.mb_attn_tma_max_cluster.argtypes = [c_int, c_int]
        lib.mb_attn_tma_max_cluster.restype = c_int
        _max_cluster[HD] = max(1, min(lib.mb_attn_tma_max_cluster(HD, 0), lib.mb_attn_tma_max_cluster(HD, 1)))
    return _max_cluster[HD]


_active_clusters = {}


def attention_tma_active_clusters(HD, cluster):
    """how many clusters of `cluster` blocks of attention_tma's decode form the device holds at the same time"""
    if (HD, cluster) not in _active_clusters:
        lib = load_library("attention_tma")
        lib.mb_attn_tma_active_clusters.argtypes = [c_int, c_int, c_int]
        lib.mb_attn_tma_active_clusters.restype = c_int
        _active_clusters[HD, cluster] = min(lib.mb_attn_tma_active_clusters(HD, r, cluster) for r in (0, 1))
    return _active_clusters[HD, cluster]


def attention_tma(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                  table, part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale, err, merge=False,
                  rope=None, cluster=0):
    """The same contract as attention_mma, with K/V tiles loaded by TMA (head sizes 64 and 128, pages of 8 to 64).
    merge: the last block of every split group merges the group's partial results and writes `out`, so no
    attention_merge is needed afterwards (only when attention_tma_merges(n_items, KV)).
    cluster = n > 1 (decode form): every sequence of the launch is cut into n splits and the blocks of a sequence and kv
    head are launched as one thread-block cluster whose results meet in shared memory (no partial buffers, no merge);
    n at most attention_tma_max_cluster(HD).
    rope = (bias or None, freqs or None, RD, pairing): the step's sequences bring ONE token each and q is the whole
    (N, (H + 2 KV) HD) output of the q/k/v product; the kernel does what rope_kv_write would have done before it (bias,
    rotation of q and k, k and v into the token's page) -- the same bits, one launch fewer.  q itself is not changed."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, part_base, table, part_o, part_ml)
    if cluster and cluster > 1:
        if not decode:
            raise KernelError("attention_tma: clusters are for the decode form")
        bias, freqs, RD, pairing = rope if rope is not None else (None, None, 0, 0)
        _cuda(bias, freqs)
        f = _fn("attention_tma", "mb_attn_tma_cluster_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_int] + [c_int] * 7 + [c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
                 _p(seq_row), _p(table), table.shape[1], int(cluster), H, KV, HD, page, num_pages, window or 0,
                 float(scale), _p(err), 1 if rope is not None else 0, _p(bias), _p(freqs), int(RD), int(pairing), _stream())
        if code == -6:
            raise KernelError("attention_tma: the driver refused the tensor map of the cache pool")
        _check(code, "attention_tma")
        return
    counters = None
    if merge:
        if not attention_tma_merges(n_items, KV):
            raise KernelError("attention_tma: more split groups than merge counters")
        key = str(q.device)
        if key not in _merge_counters:
            _merge_counters[key] = torch.zeros(MERGE_COUNTERS, dtype=torch.int32, device=q.device)
            _scratch["generation"] += 1
        counters = _merge_counters[key]
    if rope is not None:
        if not decode:
            raise KernelError("attention_tma: the rotation is folded into the decode form only")
        bias, freqs, RD, pairing = rope
        _cuda(bias, freqs)
        f = _fn("attention_tma", "mb_attn_tma_rope_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p, c_void_p,
                                                                                c_void_p, c_int, c_int, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
                 _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml), max_splits, H, KV, HD,
                 page, num_pages, window or 0, float(scale), _p(counters), _p(err), _p(bias), _p(freqs), int(RD),
                 int(pairing), _stream())
    else:
        f = _fn("attention_tma", "mb_attn_tma_bf16",
                [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_float, c_void_p, c_void_p, c_void_p])
        code = f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, 1 if decode else 0, _p(q_start),
                 _p(q_len), _p(pos0), _p(part_base), _p(seq_row), _p(table), table.shape[1], _p(part_o), _p(part_ml),
                 max_splits, H, KV, HD, page, num_pages, window or 0, float(scale), _p(counters), _p(err), _stream())
    if code == -6:
        raise KernelError("attention_tma: the driver refused the tensor map of the cache pool")
    _check(code, "attention_tma")


def attention_tc5_supports(HD, page):
    return HD in (64, 128) and page in (8, 16, 32, 64, 128)


def attention_tc5_rows():
    """packed query rows of one work item of the tcgen05 attention kernel"""
    lib = load_library("attention_tc5")
    lib.mb_attn_tc5_rows.restype = c_int
    return lib.mb_attn_tc5_rows()


def attention_tc5(q, q_stride, out, kpool, vpool, items, n_items, q_start, q_len, pos0, seq_row, table, H, KV, HD, page,
                  num_pages, window, scale, err):
    """Prompt-form attention on tcgen05: items are (sequence, tile of attention_tc5_rows() packed rows, 0, 1); head
    sizes 64 and 128."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, seq_row, table)
    f = _fn("attention_tc5", "mb_attn_tc5_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int] + [c_int] * 6 + [c_float, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
             _p(seq_row), _p(table), table.shape[1], H, KV, HD, page, num_pages, window or 0, float(scale),
             _p(err), _stream()), "attention_tc5")


def attention_tc5_diff_supports(dim, vdim, page):
    """the tcgen05 kernel's differential form: two maps of `dim` side by side are one row of vdim = 2 dim = 64 or 128"""
    return 2 * dim == vdim and attention_tc5_supports(vdim, page)


def attention_tc5_diff_rows():
    """packed query rows of one work item of the differential form (both maps of 128 rows)"""
    return 128


def attention_tc5_diff(q, out, items, n_items, q_start, q_len, pos0, seq_row, table, kpool, vpool, H, G, dim, vdim, page,
                       num_pages, chunk, scale, lam, gain, eps, err):
    """Prompt-form differential attention on tcgen05 (the result of attention_diff_simple): items are (sequence, tile of
    128 packed rows, 0, 1); q (N, H * 2 dim), kpool (pages, G, page, 2 dim), vpool (pages, G, page, vdim), vdim = 2 dim."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, seq_row, table)
    if q.dtype != torch.bfloat16 or not attention_tc5_diff_supports(dim, vdim, page):
        raise KernelError(f"attention_tc5_diff: no kernel for {q.dtype}, head sizes {dim} and {vdim}, pages of {page}")
    f = _fn("attention_tc5_diff", "mb_attn_tc5_diff_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int] + [c_int] * 6 + [c_float] * 4 + [c_void_p, c_void_p])
    _check(f(_p(q), H * vdim, _p(out), _p(kpool), _p(vpool), _p(items), n_items, _p(q_start), _p(q_len), _p(pos0),
             _p(seq_row), _p(table), table.shape[1], H, G, vdim, page, num_pages, int(chunk or 0), float(scale), float(lam),
             float(gain), float(eps), _p(err), _stream()), "attention_tc5_diff")


def attention_merge(part_o, part_ml, part_tok, n_part, out, H, HD, max_splits):
    _cuda(part_o, part_ml, part_tok, out)
    f = _fn("attention_mma", "mb_attn_merge_bf16",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(part_o), _p(part_ml), _p(part_tok), n_part, _p(out), H, HD, max_splits, _stream()), "attention_merge")


# ------------------------------------------------------------------------------------------------ sampling
def sample_params_size():
    lib = load_library("sampling")
    lib.mb_sample_params_size.restype = c_int
    return lib.mb_sample_params_size()


_sample_scratch = {}


def sample(logits, work, params, cnt, seen, n_rows, out, any_cut=True, keep_work=True):
    """logits (R, V) float32; work (n_rows, V) float32 scratch; params: uint8 tensor of n_rows packed RowParams;
    cnt (slots, V) int32 / seen (slots, V) uint8 penalty state or None; out (n_rows,) int32.  any_cut: False when no
    row has a top_k, top_p or min_p (the kernel that finds the cuts is skipped).  keep_work: leave the processed
    logits after the cuts (cut values -inf) in `work`, which costs a write of every row."""
    _cuda(logits, work, params, cnt, seen, out)
    key = str(logits.device)
    sc = _sample_scratch.get(key)
    if sc is None or sc[0].shape[0] < n_rows * 32:
        cap = max(n_rows, 64)
        sc = (torch.empty(cap * 32, dtype=torch.float32, device=logits.device),
              torch.empty(cap * 32, dtype=torch.int32, device=logits.device),
              torch.empty(cap * 2, dtype=torch.int32, device=logits.device))
        _sample_scratch[key] = sc
        _scratch["generation"] += 1
    f = _fn("sampling", "mb_sample_fast", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), _p(work), _p(params), _p(cnt), _p(seen), n_rows, logits.shape[1], _p(sc[2]), _p(sc[0]), _p(sc[1]),
             _p(work) if keep_work else None, 1 if any_cut else 0, _p(out), _stream()), "sample")


def sample_one_kernel(logits, work, params, cnt, seen, n_rows, out):
    """The same sampler as one kernel with a block per row that bisects the whole row (a millisecond for a batch at a
    vocabulary of 128k): what the entry point without allocations runs, kept callable for comparison."""
    _cuda(logits, work, params, cnt, seen, out)
    f = _fn("sampling", "mb_sample", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), _p(work), _p(params), _p(cnt), _p(seen), n_rows, logits.shape[1], _p(out), _stream()), "sample")


_argmax_scratch = {}


def argmax(logits, out):
    """out[r] = the lowest index of the maximum of row r"""
    _cuda(logits, out)
    n = logits.shape[0]
    key = str(logits.device)
    sc = _argmax_scratch.get(key)
    if sc is None or sc[0].shape[0] < n * 32:
        sc = (torch.empty(max(n, 64) * 32, dtype=torch.float32, device=logits.device),
              torch.empty(max(n, 64) * 32, dtype=torch.int32, device=logits.device))
        _argmax_scratch[key] = sc
        _scratch["generation"] += 1
    f = _fn("sampling", "mb_argmax", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_p(logits), n, logits.shape[1], _p(sc[0]), _p(sc[1]), _p(out), _stream()), "argmax")


def penalty_fill(cnt_row, seen_row, tokens, n_prompt, n_total, V):
    _cuda(cnt_row, seen_row, tokens)
    f = _fn("sampling", "mb_penalty_fill", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_p(cnt_row), _p(seen_row), _p(tokens), n_prompt, n_total, V, _stream()), "penalty_fill")


# ------------------------------------------------------------------------------------------------ tracing
def logit_trace(logits, out):
    """logits (R, V) float32 contiguous -> out (R, 2) int32: per row the order-independent hash
    sum(bits(lg[v]) * (2 v + 1)) mod 2^32 and the bits of the float32 gap between the two largest logits
    (src/mashbox/runtime/engine.py:80-89)."""
    _cuda(logits, out)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("logit_trace: float32 contiguous logits only")
    f = _fn("trace", "mb_logit_trace", [c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(f(_p(logits), logits.shape[0], logits.shape[1], _p(out), _stream()), "logit_trace")


def read_logit_trace(pairs):
    """int32 (R, 2) as logit_trace writes it (any device or a numpy array) -> [(hash, gap)] with hash in 0..2^32-1"""
    import numpy as np
    a = np.ascontiguousarray(pairs.cpu().numpy() if hasattr(pairs, "cpu") else pairs, dtype=np.int32).reshape(-1, 2)
    return [(int(h), float(g)) for h, g in zip(a[:, 0].view(np.uint32), a[:, 1].copy().view(np.float32))]


# ------------------------------------------------------------------------------------------------ layer norm on outputs
def ln_add(x, y1, w, b, eps, copy=None, y2=None, s1=1.0, s2=1.0):
    """x (N, D) float32 += layer_norm(s1 y1 + s2 y2) * w + b, row by row (y2 None: y1 alone); y1, y2 in the activation
    dtype; copy: the new x in the activation dtype"""
    _cuda(x, y1, y2, w, b, copy)
    N, D = x.shape
    f = _fn("layernorm", "mb_ln_add_" + _suffix(y1.dtype),
            [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(y1), _p(y2), float(s1), float(s2), _p(w), _p(b), float(eps), _p(copy), N, D, _stream()), "ln_add")


def layer_norm(x, rows, w, b, eps, out):
    """out = layer_norm(x[rows]) * w + b (rows None: every row); x (N, D) float32, out in the activation dtype"""
    _cuda(x, rows, w, b, out)
    f = _fn("layernorm", "mb_layer_norm_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    _check(f(_p(x), _p(rows), _p(w), _p(b), float(eps), _p(out), out.shape[0], x.shape[1], _stream()), "layer_norm")


def to_rows(x, out):
    """out = x (float32) in the activation dtype"""
    _cuda(x, out)
    f = _fn("layernorm", "mb_to_rows_" + _suffix(out.dtype), [c_void_p, c_void_p, c_ll, c_void_p])
    _check(f(_p(x), _p(out), x.numel(), _stream()), "to_rows")


def glu_clamped(gu, out, limit, alpha=1.702, shift=1.0):
    """gu (N, 2F) = [gate | up] -> out (N, F) = g sigmoid(alpha g) (u + shift) with g = min(gate, limit),
    u = clamp(up, -limit, limit); limit None: no clamps"""
    _cuda(gu, out)
    N, F = out.shape
    f = _fn("elementwise", "mb_glu_clamped_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(_p(gu), _p(out), N, F, float(limit or 0.0), float(alpha), float(shift), _stream()), "glu_clamped")


# ------------------------------------------------------------------------------------------------ gated recurrences
def gla_gates(rows, z, zb, tau, q, k, v, g, H, dim, vdim):
    """rows (N, >= 2 H dim + H vdim) = [q | k | v | ..] in the activation dtype, z (N, H dim) float32 decay logits, zb
    their bias -> float32 q (times dim^-1/2), k (N, H dim), v (N, H vdim), g = sigmoid(z + zb)^(1 / tau)"""
    _cuda(rows, z, zb, q, k, v, g)
    f = _fn("gated_scan", "mb_gla_gates_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_float] + [c_void_p] * 4 + [c_int] * 4 + [c_void_p])
    _check(f(_p(rows), rows.stride(0), _p(z), _p(zb), 1.0 / float(tau), _p(q), _p(k), _p(v), _p(g), rows.shape[0], H, dim,
             vdim, _stream()), "gla_gates")


def ssd_gates(xbc, conv_bias, dt, dt_bias, A_log, q, k, v, g, H, G, P, NS):
    """xbc (N, H P + 2 G NS) = [x | B | C] after the convolution (activation dtype), dt (N, H) float32 raw step sizes ->
    float32 v = softplus(dt + dt_bias) silu(x + bias) (N, H P), k = silu(B + bias), q = silu(C + bias) (N, G NS),
    g = exp(-exp(A_log) softplus(dt + dt_bias)) (N, H)"""
    _cuda(xbc, conv_bias, dt, dt_bias, A_log, q, k, v, g)
    f = _fn("gated_scan", "mb_ssd_gates_" + _suffix(xbc.dtype), [c_void_p] * 9 + [c_int] * 5 + [c_void_p])
    _check(f(_p(xbc), _p(conv_bias), _p(dt), _p(dt_bias), _p(A_log), _p(q), _p(k), _p(v), _p(g), xbc.shape[0], H, G, P, NS,
             _stream()), "ssd_gates")


def ssd_out(o, xbc, conv_bias, D, z, w, out, H, P, parts, eps):
    """out = rms over each of `parts` equal stretches of ((o + D x) silu(z)), times w: o (N, H P) float32 from the
    recurrence, x = silu(xbc[:, :H P] + bias), z (N, H P) a view of the gate's logits, out in the activation dtype"""
    _cuda(o, xbc, conv_bias, D, z, w, out)
    f = _fn("gated_scan", "mb_ssd_out_" + _suffix(out.dtype),
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 4
            + [c_float, c_void_p])
    _check(f(_p(o), _p(xbc), xbc.stride(0), _p(conv_bias), _p(D), _p(z), z.stride(0), _p(w), _p(out), o.shape[0], H, P,
             parts, float(eps), _stream()), "ssd_out")


def gated_scan(q, k, v, g, o, state, seq, H, G, dim, vdim, per_head):
    """S <- decay S + k v^T, o = S^T q per head and token, tokens of a sequence in order.  q, k (N, G dim), v (N, H vdim),
    o (N, H vdim) float32; g (N, H dim) a decay per key channel, or (N, H) with per_head; state (slots, H dim vdim)
    float32 (a view: slots state.stride(0) apart); seq = (q_start, q_len, state_slot) int32 device arrays"""
    _cuda(q, k, v, g, o, state, *seq)
    f = _fn("gated_scan", "mb_gated_scan", [c_void_p] * 6 + [c_ll] + [c_void_p] * 3 + [c_int] * 7 + [c_void_p])
    S = seq[0].shape[0]
    # which layout of the state over threads: by the step's tokens per sequence (from the lengths of the arrays alone)
    _check(f(_p(q), _p(k), _p(v), _p(g), _p(o), _p(state), state.stride(0), *[_p(t) for t in seq], S, H, G,
             dim, vdim, 1 if per_head else 0, 1 if q.shape[0] > 4 * S else 0, _stream()), "gated_scan")


# ------------------------------------------------------------------------------------------------ normed, rotated heads
def norm_rope_kv_write(rows, qw, kw, eps, freqs, RD, pairing, gain, positions, tok_row, table, kpool, vpool, H, KV, DK,
                       DV, page, num_pages, err):
    """rows (N, >= (H + KV) DK + KV DV) = [q | k | v | ..]: every q and k head divided by its root mean square and
    multiplied by qw / kw (DK values; None: no norm), its first RD values rotated by the token's position (freqs (RD/2,)
    float32 or None; pairing 0 adjacent, 1 halves; cos and sin times gain); q back in place, k and v into the pages:
    kpool (pages, KV, page, DK), vpool (pages, KV, page, DV); both None: q only"""
    _cuda(rows, qw, kw, freqs, positions, tok_row, table, kpool, vpool)
    f = _fn("rotary_rows", "mb_norm_rope_kv_write_" + _suffix(rows.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
             c_int, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p, c_void_p])
    _check(f(_p(rows), rows.stride(0), _p(qw), _p(kw), float(eps), _p(freqs), int(RD), int(pairing), float(gain),
             _p(positions), _p(tok_row), _p(table), table.shape[1], _p(kpool), _p(vpool), rows.shape[0], H, KV, DK, DV, page,
             num_pages, _p(err), _stream()), "norm_rope_kv_write")


def latent_rope(q, q_head, q_off, qa, qa_head, qa_off, rows, kr_off, pool, pool_off, freqs, RD, W, pairing, gain,
                positions, tok_row, table, H, page, num_pages, err):
    """The strips of W values that latent attention rotates (the first RD of them turn): of every query head, q (N, H
    q_head) at q_off, into qa (N, H qa_head) at qa_off; of the token's shared key strip, rows[:, kr_off:], into the
    position's cache row at pool_off (pool (pages, 1, page, row); None: a layer that borrows its cache)"""
    _cuda(q, qa, rows, pool, freqs, positions, tok_row, table)
    f = _fn("rotary_rows", "mb_latent_rope_" + _suffix(q.dtype),
            [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
             c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p])
    _check(f(_p(q), q.stride(0), q_head, q_off, _p(qa), qa_head, qa_off, _p(rows), rows.stride(0), kr_off, _p(pool),
             pool.shape[-1] if pool is not None else 0, pool_off, _p(freqs), int(RD), int(W), int(pairing), float(gain),
             _p(positions), _p(tok_row), _p(table), table.shape[1], q.shape[0], H, page, num_pages, _p(err), _stream()),
           "latent_rope")


def attention_general(q, q_stride, out, positions, tok_seq, table, kpool, vpool, H, KV, DK, DV, page, num_pages, window,
                      scale, err, softcap=None, sinks=None, gate=None):
    """The plain paged attention kernel in its general form: keys of DK and values of DV values (the pools' rows may be
    wider: their last dimension is the distance between two positions), scores capped by softcap tanh(s / softcap), a
    sink per query head in the denominator (sinks (H,) float32), the result of head h times sigmoid(gate[n, h])"""
    _cuda(q, out, positions, tok_seq, table, kpool, vpool, sinks, gate)
    N = out.shape[0]
    f = _fn("attention_simple", "mb_attn_simple_ext_" + _suffix(out.dtype),
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p] + [c_int] * 10
            + [c_float, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(positions), _p(tok_seq), _p(table), table.shape[1], _p(kpool), _p(vpool), N, H,
             KV, DK, DV, kpool.shape[-1], vpool.shape[-1], page, num_pages, window or 0, float(scale),
             float(softcap or 0.0), _p(sinks), _p(gate), gate.stride(0) if gate is not None else 0, _p(err), _stream()),
           "attention_general")


def attention_general_mma_supports(DK, DV):
    """the tensor-core form of the general attention takes these key and value widths (bfloat16 only)"""
    return DK % 16 == 0 and DV % 16 == 0 and 16 <= DK <= 256 and 16 <= DV <= 256


def _general_mma_library(DK, DV):
    from .build import variant
    return variant(f"attention_general_mma_{DK}_{DV}", "attention_general_mma.cu", [f"-DGA_DK={DK}", f"-DGA_DV={DV}"])


def attention_general_mma(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                          table, part_o, part_ml, max_splits, H, KV, DK, DV, page, num_pages, window, scale, err,
                          softcap=None, sinks=None, gate=None):
    """attention_general on tensor cores (bfloat16): items are (sequence, row tile, split, splits) quadruples of the
    prompt form (tiles of 64 packed rows) or, with decode, of the decode form (at most 16); split items leave partial
    sums in part_o / part_ml for attention_general_merge.  Compiled for the pair (DK, DV) the first time it is asked for."""
    _cuda(q, out, kpool, vpool, items, q_start, q_len, pos0, part_base, seq_row, table, part_o, part_ml, sinks, gate)
    if out.dtype != torch.bfloat16 or not attention_general_mma_supports(DK, DV):
        raise KernelError(f"attention_general_mma: no kernel for {out.dtype} with widths {DK} and {DV}")
    f = _fn(_general_mma_library(DK, DV), "mb_attn_general_bf16",
            [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int] + [c_void_p] * 6 + [c_int]
            + [c_void_p, c_void_p] + [c_int] * 8 + [c_float, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(f(_p(q), q_stride, _p(out), _p(kpool), _p(vpool), kpool.shape[-1], vpool.shape[-1], _p(items), int(n_items),
             1 if decode else 0, _p(q_start), _p(q_len), _p(pos0), _p(part_base), _p(seq_row), _p(table), table.shape[1],
             _p(part_o), _p(part_ml), max_splits, H, KV, DK, DV, page, num_pages, window or 0, float(scale),
             float(softcap or 0.0), _p(sinks), _p(gate), gate.stride(0) if gate is not None else 0, _p(err), _stream()),
           "attention_general_mma")


def attention_general_merge(part_o, part_ml, part_tok, n_part, out, H, DK, DV, max_splits, sinks=None, gate=None):
    """adds up the splits of the tokens whose keys were cut (part_tok: (token, splits) pairs), sink and gate included"""
    _cuda(part_o, part_ml, part_tok, out, sinks, gate)
    f = _fn(_general_mma_library(DK, DV), "mb_attn_general_merge_bf16",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_p(part_o), _p(part_ml), _p(part_tok), n_part, _p(out), H, DV, max_splits, _p(sinks), _p(gate),
             gate.stride(0) if gate is not None else 0, _stream()), "attention_general_merge")
