"""TEST INFRASTRUCTURE ONLY -- CPU restatement (torch CPU ops + numpy bit tricks) of the
chunked XMC classifier train step of xmc-aalto/elmo.

Nothing in the product path may import this file: only tests/, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of bench.py do, as the checker or as the timed
CPU baseline.

What is restated (reference file:line, paths relative to the reference's root):

* ``chunked_step``      -- src/xmc_classifiers/chunked.py:75-133  (XMCBCECHUNKEDLayer)
* ``fp8_chunked_step``  -- src/xmc_classifiers/chunked_fp8xmc_clf.py:81-123 (real and
                           simulated FP8), with its kernels
    - ``large_k_matmul``  src/triton_kernels/matmul_kernel.py:204-239,342-353
    - ``matmul_update``   src/triton_kernels/fuse_kernel.py:63-131
    - ``fakefp8 update``  src/triton_kernels/fuse_kernel.py:134-199 +
                          chunked_fp8xmc_clf.py:115-116
    - ``kahan update``    src/triton_kernels/fuse_kernel.py:202-287
* ``sgd`` elementwise   -- src/triton_kernels/stochastic_rounding_kernel.py:65-99
* ``bce_sum_loss``      -- src/xmc_classifiers/chunked.py:57-72
* ``fp8_padded_labels`` -- src/xmc_classifiers/chunked_fp8xmc_clf.py:26-28
* ``forward_logits``    -- chunked.py:48-53, chunked_fp8xmc_clf.py:45-60

Parity pins: the reference ships no golden vectors or executable tests.  This oracle is
pinned against outputs of the reference itself (tests/test_oracle_golden.py and
tests/test_oracle_golden_gpu.py replay the fixtures):
  * imported unmodified on CPU (tests/golden/make_golden.py):
    - XMCBCECHUNKEDLayer in float32 end to end (W', grad_input);
    - XMCBCECHUNKEDLayer in bfloat16 with only the Triton ``sgd_update`` launcher replaced
      by a round-to-nearest torch statement;
    - ``torch._scaled_mm`` e4m3 forward and ``xfc_forward`` of Fp8XMCBCEChunkedLayer;
    - ``_compute_loss``;
  * run unmodified on a B200 (tests/golden/make_golden_gpu.py, from the staging copy that
    oracle/make_ref.py makes): the Triton kernels ``stochastic_rounding`` / ``large_k_matmul`` /
    ``matmul_update`` / ``kahan_matmul_update`` / ``fakefp8_matmul_update`` / ``sgd_update`` and two
    steps each of Fp8XMCBCEChunkedLayer (real and simulated), Fp8XMCBCEChunkedHeadKahanLayer and
    bfloat16 XMCBCECHUNKEDLayer.  With rounding mode 'sr_triton' (below) the oracle reproduces
    the reference's stochastically rounded weights bit for bit up to accumulation-order effects.

Rounding modes
  'rn'     round-to-nearest-even of the fp32 update (the value the authors compare against in
           fuse_kernel.py:309-310); the reference itself has no such switch.
  'sr'     this build's stochastic rounding: exact SR on the target grid (e4m3 including its
           subnormals, or bf16) driven by 16 Philox bits per element (oracle/philox.py).
  'sr_ref' the reference's bit trick (fuse_kernel.py:28-36) driven by the same 16 bits widened
           to 20; kept to document that it is biased below 2^-6.
  'sr_triton' the reference's own stochastic rounding, stream included: the bit trick driven by
           ``tl.randint(seed, offset)`` with the per-launch seed the reference draws on the host and
           offsets restarting at 0 in every updated tensor (fuse_kernel.py:107, chunked_fp8xmc_clf.py:113).
           Used only to pin this file against the reference's GPU outputs.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import philox

E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0


# ----------------------------------------------------------------------------------------------
# small helpers
# ----------------------------------------------------------------------------------------------
def fp8_padded_labels(num_labels: int, num_chunks: int) -> Tuple[int, int]:
    """(L', L_i) of the FP8 classes: chunked_fp8xmc_clf.py:26-28 (adds a full 16*nc when aligned)."""
    lp = num_labels + 16 * num_chunks - num_labels % (16 * num_chunks)
    li = lp // num_chunks
    assert li % 16 == 0
    return lp, li


def _bf16(x: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 (RNE) and return it as fp32 values."""
    return x.to(torch.bfloat16).to(torch.float32)


def cast_e4m3_sat(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 RNE, saturating at +-448 (torch's own cast gives NaN above 464).

    The CUDA library saturates (``__NV_SATFINITE``); for |x| < 464 both agree bit for bit.
    """
    x = x.to(torch.float32)
    return torch.where(torch.isnan(x), x, x.clamp(-E4M3_MAX, E4M3_MAX)).to(E4M3)


def positives_mask(labels: torch.Tensor, lo: int, hi: int, bsz: int) -> torch.Tensor:
    """Dense 0/1 mask [hi-lo, bsz] (label-major) of the positives whose label id falls in
    [lo, hi): chunked_fp8xmc_clf.py:124-126 + :108.  Duplicate pairs count once (index_put
    without accumulate)."""
    rows = labels[:, 0].long()
    cols = labels[:, 1].long()
    m = (cols >= lo) & (cols < hi)
    y = torch.zeros(hi - lo, bsz, dtype=torch.bool)
    y[cols[m] - lo, rows[m]] = True
    return y


def bce_sum_loss(logits: torch.Tensor, y: torch.Tensor) -> float:
    """Summed BCE-with-logits, chunked.py:57-72:  sum max(z,0) - sum_pos z + sum log(1+e^-|z|).

    Evaluated in float64 on the (already rounded) logits; y is a boolean mask of the same shape
    (binary targets: a duplicated pair counts once).
    """
    z = logits.to(torch.float64)
    return float(z.clamp(min=0).sum() - z[y].sum() + torch.log1p(torch.exp(-z.abs())).sum())


# ----------------------------------------------------------------------------------------------
# rounding of the fp32 update onto the weight grid
# ----------------------------------------------------------------------------------------------
def _f32_bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def sr_e4m3_exact(w: np.ndarray, r16: np.ndarray) -> np.ndarray:
    """Exact stochastic rounding of fp32 ``w`` to the e4m3 grid with 16 random bits.

    |w| is clamped to 448 first (NaN stays NaN).  For |w| >= 2^-6 the grid step is 2^(e-3):
    add ``r16 << 4`` into the low 20 mantissa bits and truncate them (the reference's trick,
    fuse_kernel.py:28-36).  Below 2^-6 the e4m3 grid is uniform with step 2^-9, which the bit
    trick does not see (its final convert re-rounds to nearest); adding 2^-6 first moves the
    value into the binade [2^-6, 2^-5) whose 3-bit step is exactly 2^-9, and subtracting it
    afterwards is exact.  The sign of w is kept, also when the result is zero (as the reference's
    trick does).  The CUDA kernel reaches the same bits by scaling with 2^-120 into fp32's own
    subnormal range.  Result is returned as fp32 values on the e4m3 grid.
    """
    w = np.asarray(w, dtype=np.float32)
    nan = np.isnan(w)
    a = np.minimum(np.abs(w), np.float32(E4M3_MAX))
    small = a < np.float32(2.0 ** -6)
    y = np.where(small, a + np.float32(2.0 ** -6), a).astype(np.float32)
    bits = _f32_bits(y) + (np.asarray(r16, dtype=np.uint32) << np.uint32(4))
    bits &= np.uint32(0xFFF00000)
    y = bits.view(np.float32)
    y = np.where(small, y - np.float32(2.0 ** -6), y).astype(np.float32)
    y = np.minimum(y, np.float32(E4M3_MAX))
    out = np.copysign(y, w).astype(np.float32)
    out[nan] = np.nan
    return out


def sr_e4m3_reference_trick(w: np.ndarray, r20: np.ndarray) -> np.ndarray:
    """fuse_kernel.py:28-36 verbatim: add 20 random bits, clear them, convert RNE to e4m3."""
    bits = _f32_bits(w) + np.asarray(r20, dtype=np.uint32)
    bits &= np.uint32(0xFFF00000)
    t = torch.from_numpy(bits.view(np.float32).copy())
    return cast_e4m3_sat(t).to(torch.float32).numpy()


def sr_bf16(w: np.ndarray, r16: np.ndarray) -> np.ndarray:
    """fuse_kernel.py:10-17 / stochastic_rounding_kernel.py:10-17: add 16 random bits to the
    fp32 pattern, clear the low 16.  Exact SR on the bf16 grid (subnormals included)."""
    bits = _f32_bits(w) + np.asarray(r16, dtype=np.uint32)
    bits &= np.uint32(0xFFFF0000)
    return bits.view(np.float32).copy()


def sr_triton(w: np.ndarray, seed: int, kind: str, first_offset: int = 0) -> torch.Tensor:
    """The reference's stochastic-rounding helpers with their own random stream
    (fuse_kernel.py:10-17,28-44; stochastic_rounding_kernel.py:10-27): element i of the flattened
    tensor draws ``tl.randint(seed, first_offset + i)``.
      kind 'e4m3'    + (r & 0xFFFFF), clear 20 bits, convert to e4m3 (Triton's fp32->e4m3 convert on
                     sm_100: round-to-nearest-even, saturating to +-448 -- pinned by the fixture)
      kind 'bf16'    + (r & 0xFFFF), clear 16 bits, convert to bf16 (exact)
      kind 'fakefp8' + (r & 0xFFFFF), clear 20 bits, convert to bf16 (exact)
    Returns a tensor of the target dtype with the shape of ``w``."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    offs = np.arange(first_offset, first_offset + w.size, dtype=np.int64).reshape(w.shape)
    r = philox.triton_randint(seed, offs)
    if kind == 'bf16':
        bits = (_f32_bits(w) + (r & np.uint32(0xFFFF))) & np.uint32(0xFFFF0000)
        return torch.from_numpy(bits.view(np.float32).copy()).to(torch.bfloat16)
    bits = (_f32_bits(w) + (r & np.uint32(0xFFFFF))) & np.uint32(0xFFF00000)
    t = torch.from_numpy(bits.view(np.float32).copy())
    if kind == 'fakefp8':
        return t.to(torch.bfloat16)
    assert kind == 'e4m3'
    return cast_e4m3_sat(t)


_CLIB = False


def _c_lib():
    """oracle/sr_philox.c compiled (same definitions as the numpy statements above, only faster);
    None when gcc is unavailable -- the numpy path is then used."""
    global _CLIB
    if _CLIB is False:
        try:
            import ctypes as C
            from . import build_c
            lib = C.CDLL(build_c.build())
            for name in ("oracle_sr_e4m3", "oracle_sr_bf16"):
                getattr(lib, name).argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                               C.c_void_p]
                getattr(lib, name).restype = None
            lib.oracle_sr_bits16.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
            lib.oracle_sr_bits16.restype = None
            _CLIB = lib
        except Exception:
            _CLIB = None
    return _CLIB


def round_update(w32: torch.Tensor, w_dtype: torch.dtype, rounding: str,
                 seed: int, step: int, first_elem: int) -> torch.Tensor:
    """Round the fp32 updated weights ``w32`` [rows, d] to ``w_dtype``.

    ``first_elem`` is the global flat index (label_row * d) of w32[0, 0]; the random bits of
    element (r, c) come from philox.sr_bits16(first_elem + r*d + c, seed, step).
    """
    if rounding == 'rn':
        if w_dtype == E4M3:
            return cast_e4m3_sat(w32)
        return w32.to(w_dtype)
    if rounding == 'sr_triton':     # here ``seed`` is the launch's host-drawn seed, ``first_elem`` the in-tensor offset
        wn = w32.detach().to(torch.float32).contiguous().numpy()
        return sr_triton(wn, seed, 'e4m3' if w_dtype == E4M3 else 'bf16', first_elem)
    n = w32.numel()
    clib = _c_lib()
    if clib is not None and rounding == 'sr' and w_dtype in (E4M3, torch.bfloat16):
        src = w32.detach().to(torch.float32).contiguous()
        out = torch.empty_like(src)
        fn = clib.oracle_sr_e4m3 if w_dtype == E4M3 else clib.oracle_sr_bf16
        fn(src.data_ptr(), n, int(first_elem), int(seed) & (2 ** 64 - 1), int(step) & (2 ** 64 - 1),
           out.data_ptr())
        return out.to(w_dtype)                          # exact: values already on the grid
    idx = np.arange(first_elem, first_elem + n, dtype=np.uint64).reshape(w32.shape)
    r16 = philox.sr_bits16(idx, seed, step)
    wn = w32.detach().to(torch.float32).contiguous().numpy()
    if w_dtype == E4M3:
        if rounding == 'sr':
            out = sr_e4m3_exact(wn, r16)
        elif rounding == 'sr_ref':
            out = sr_e4m3_reference_trick(wn, r16 << np.uint32(4))
        else:
            raise ValueError(rounding)
        return torch.from_numpy(out).to(E4M3)           # exact: values already on the grid
    if w_dtype == torch.bfloat16:
        return torch.from_numpy(sr_bf16(wn, r16)).to(torch.bfloat16)
    raise ValueError(w_dtype)


def fused_update(w: torch.Tensor, acc: torch.Tensor, lr: float, wd: float = 0.0) -> torch.Tensor:
    """fp32 value ``w - lr*(acc + wd*w)`` with one rounding (the kernels contract it into an
    FMA: fuse_kernel.py:105 ``weights - lr*acc``).  lr and wd are fp32 scalars."""
    lr32 = float(np.float32(lr)); wd32 = float(np.float32(wd))
    w64 = w.to(torch.float64)
    a64 = acc.to(torch.float64)
    if wd32 != 0.0:
        a64 = (a64 + wd32 * w64).to(torch.float32).to(torch.float64)
    return (w64 - lr32 * a64).to(torch.float32)


# ----------------------------------------------------------------------------------------------
# kernels of the FP8 path
# ----------------------------------------------------------------------------------------------
def scaled_mm_e4m3(w8: torch.Tensor, x8: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``torch._scaled_mm(W_i, X8^T, scale 1, 1, out bf16)`` of chunked_fp8xmc_clf.py:101-102:
    e4m3 x e4m3 products accumulated in fp32, optionally times a per-tensor scale, rounded to
    bf16.  Returns logits^T [L_i, B] as bf16."""
    z = w8.to(torch.float32) @ x8.to(torch.float32).t()
    if scale != 1.0:
        z = z * float(np.float32(scale))
    return z.to(torch.bfloat16)


def large_k_matmul(g: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """matmul_kernel.py:204-239: C[m,n] fp32 = g^T @ w with both operands rounded to bf16 and
    fp32 accumulation (the kernel's atomic order is unspecified; so is ours here)."""
    return _bf16(g.to(torch.float32)).t() @ _bf16(w.to(torch.float32))


def matmul_acc(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """The accumulator of fuse_kernel.py:84-96: sum_k bf16(g[m,k]) * bf16(x[k,n]) in fp32."""
    return _bf16(g.to(torch.float32)) @ _bf16(x.to(torch.float32))


# ----------------------------------------------------------------------------------------------
# full steps
# ----------------------------------------------------------------------------------------------
def fp8_chunked_step(w_chunks: Sequence[torch.Tensor], x: torch.Tensor, labels: torch.Tensor,
                     lr: float, *, simulated: bool = False, rounding: str = 'rn',
                     seed: int = 0, step: int = 0, w_scale: float = 1.0,
                     label_offset: int = 0, compute_loss: bool = False,
                     kahan: Optional[torch.Tensor] = None,
                     chunk_seeds: Optional[Sequence[int]] = None, fp8_dw: bool = False,
                     ) -> Tuple[List[torch.Tensor], torch.Tensor, float]:
    """One ``Fp8XMCBCEChunkedLayer.xfc_forward_backward`` (chunked_fp8xmc_clf.py:81-123).

    w_chunks : list of e4m3 [L_i, d] tensors (stored value * w_scale = real weight)
    x        : bf16 [B, d];  labels: int32 [nnz, 2] (row, global label id)
    label_offset : global id of w_chunks[0][0] (label-range sharding); also the origin of the
                   Philox element index, so sharded and unsharded runs draw the same bits.
    kahan    : optional compensation buffer for rows [0, num_head) of chunk 0
               (chunked_head_kahan_fp8xmc_clf.py:127-131), bf16 or e5m2; updated in place.
    fp8_dw   : NOT the reference's arithmetic -- the build's optional FP8-operand dW contraction:
               ``acc = e4m3(G * 256) . e4m3(X) / 256`` instead of bf16 operands (fuse_kernel.py:88-92);
               grad_X keeps bf16 operands.  Restated here so that the variant has an oracle of its own.
    chunk_seeds : rounding 'sr_triton' only -- the seed the reference draws on the host for each
               chunk (chunked_fp8xmc_clf.py:113); offsets restart at 0 in every updated tensor.
    Returns (new chunks, grad_X fp32 [B, d] (not yet cast to bf16), loss).
    """
    assert x.dtype == torch.bfloat16
    bsz, d = x.shape
    x32 = x.to(torch.float32)
    x8 = cast_e4m3_sat(x32)
    s32 = float(np.float32(w_scale))
    lr_eff = float(np.float32(np.float32(lr) / np.float32(w_scale)))
    grad_x = torch.zeros(bsz, d, dtype=torch.float32)
    new_chunks = []
    loss = 0.0
    row0 = 0
    for w8 in w_chunks:
        li = w8.shape[0]
        lo = label_offset + row0
        w32 = w8.to(torch.float32)
        if simulated:
            zt = (w32 @ x32.t())                               # :98-99, bf16 GEMM, fp32 accumulate
            if s32 != 1.0:
                zt = zt * s32
            zt = zt.to(torch.bfloat16)
        else:
            zt = scaled_mm_e4m3(w8, x8, w_scale)               # :101-102
        y = positives_mask(labels, lo, lo + li, bsz)           # :105
        if compute_loss:
            loss += bce_sum_loss(zt, y)
        g = torch.sigmoid(zt)                                  # :107  (bf16 in, bf16 out)
        g = torch.where(y, g - 1.0, g)                         # :108  (bf16 arithmetic)
        gx = large_k_matmul(g, w32)                            # :109-112
        grad_x += gx * s32 if s32 != 1.0 else gx
        if fp8_dw:
            g8 = cast_e4m3_sat(g.to(torch.float32) * 256.0).to(torch.float32)
            acc = (g8 @ x8.to(torch.float32)) / 256.0
        else:
            acc = matmul_acc(g, x32)                           # fuse_kernel.py:84-96 (bf16 embed)
        first = lo * d
        sd = seed
        tri = rounding == 'sr_triton'
        if tri:
            sd, first = int(chunk_seeds[len(new_chunks)]), 0
        if kahan is not None and row0 == 0:
            nh = kahan.shape[0]
            k32 = kahan.to(torch.float32)
            wk = fused_update(w32[:nh] + k32, acc[:nh], lr_eff)            # fuse_kernel.py:257-258
            head = round_update(wk, E4M3, rounding, sd, step, first)
            knew = k32 + w32[:nh] - head.to(torch.float32) - lr_eff * acc[:nh]   # :267
            kahan.copy_(knew.to(kahan.dtype))
            # the tail is a launch of its own with the same seed: its offsets restart at 0
            # (chunked_head_kahan_fp8xmc_clf.py:131)
            tail = round_update(fused_update(w32[nh:], acc[nh:], lr_eff), E4M3, rounding,
                                sd, step, 0 if tri else first + nh * d)
            new = torch.cat([head, tail], 0)
        elif simulated and tri:
            # fuse_kernel.py:134-182 on the bf16 copy, then chunked_fp8xmc_clf.py:116 casts it back
            w_upd = fused_update(w32, acc, lr_eff)
            w16 = sr_triton(w_upd.numpy(), sd, 'fakefp8', 0)
            new = w16.to(E4M3)
        else:
            w_upd = fused_update(w32, acc, lr_eff)             # fuse_kernel.py:105
            new = round_update(w_upd, E4M3, rounding, sd, step, first)
        new_chunks.append(new)
        row0 += li
    return new_chunks, grad_x, loss


def chunked_step(w: torch.Tensor, x: torch.Tensor, labels: torch.Tensor, lr: float, *,
                 num_chunks: int, wd: float = 0.0, rounding: str = 'rn', seed: int = 0,
                 step: int = 0, label_offset: int = 0, compute_loss: bool = False,
                 chunk_seeds: Optional[Sequence[int]] = None,
                 ) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """One ``XMCBCECHUNKEDLayer.xfc_forward_backward`` (chunked.py:75-133).

    fp32 weights: plain SGD with weight decay (:122-124).  bf16 weights: dW is materialised in
    bf16 (:119) and ``_sgd`` applies ``W - dW*lr`` without weight decay
    (stochastic_rounding_kernel.py:82-83,91-99 ignore wd), then rounds per ``rounding``.
    Returns (W', grad_X fp32 [B, d], loss)."""
    L, d = w.shape
    bsz = x.shape[0]
    dt = w.dtype
    xd = x.to(dt)
    chunk = (L + num_chunks - 1) // num_chunks                 # :30
    grad_x = torch.zeros(bsz, d, dtype=torch.float32)
    w_new = w.clone()
    loss = 0.0
    for c in range(num_chunks):
        s, e = c * chunk, min((c + 1) * chunk, L)
        if s >= e:
            continue
        wc = w[s:e]
        z = (xd.to(torch.float32) @ wc.to(torch.float32).t()).to(dt)        # :101
        y = positives_mask(labels, label_offset + s, label_offset + e, bsz).t()
        if compute_loss:
            loss += bce_sum_loss(z, y)
        g = torch.sigmoid(z)                                   # :112
        g = torch.where(y, g - 1.0, g)                         # :113
        grad_x += g.to(torch.float32) @ wc.to(torch.float32)   # :116
        dw = (g.to(torch.float32).t() @ xd.to(torch.float32)).to(dt)        # :119
        if dt == torch.float32 or dt == torch.float16:
            dw = dw + wd * wc                                  # :123
            w_new[s:e] = wc - lr * dw                          # :124
        else:
            lr32 = float(np.float32(lr))
            upd = (wc.to(torch.float64) - dw.to(torch.float64) * lr32).to(torch.float32)
            if rounding == 'sr_triton':                        # chunked.py:126-127: one host seed per chunk
                w_new[s:e] = round_update(upd, dt, rounding, int(chunk_seeds[c]), step, 0)
            else:
                w_new[s:e] = round_update(upd, dt, rounding, seed, step, (label_offset + s) * d)
    return w_new, grad_x, loss


def forward_logits(w_chunks: Sequence[torch.Tensor], x: torch.Tensor, *, simulated: bool = False,
                   w_scale: float = 1.0, num_labels: Optional[int] = None) -> torch.Tensor:
    """``xfc_forward`` (chunked_fp8xmc_clf.py:45-60; chunked.py:48-53 for a single bf16 'chunk'):
    logits [B, num_labels] bf16, padding rows sliced off."""
    outs = []
    for wc in w_chunks:
        if wc.dtype == E4M3 and not simulated:
            x8 = x if x.dtype == E4M3 else cast_e4m3_sat(x.to(torch.float32))
            outs.append(scaled_mm_e4m3(wc, x8, w_scale).t())
        else:
            z = x.to(torch.bfloat16).to(torch.float32) @ wc.to(torch.float32).t()
            if w_scale != 1.0:
                z = z * float(np.float32(w_scale))
            outs.append(z.to(torch.bfloat16))
    out = torch.cat(outs, 1)
    return out if num_labels is None else out[:, :num_labels]


def topk_logits(w_chunks, x, k: int, **kw) -> Tuple[torch.Tensor, torch.Tensor]:
    """evaluate.py:158-159: ``xfc_forward`` followed by ``torch.topk`` (here sorted, ties to the
    lower label id so that the result is unique)."""
    z = forward_logits(w_chunks, x, **kw).to(torch.float32)
    order = torch.argsort(-z, dim=1, stable=True)[:, :k]
    return torch.gather(z, 1, order), order.to(torch.int32)


# ----------------------------------------------------------------------------------------------
# label-range sharding (new in the build; defined as "equal to the unsharded step")
# ----------------------------------------------------------------------------------------------
def shard_bounds(num_rows: int, world: int, align: int = 1) -> List[Tuple[int, int]]:
    """Contiguous label ranges: rank r owns [r*ceil(L/g), min((r+1)*ceil(L/g), L))."""
    per = (num_rows + world - 1) // world
    per = (per + align - 1) // align * align
    return [(min(r * per, num_rows), min((r + 1) * per, num_rows)) for r in range(world)]
