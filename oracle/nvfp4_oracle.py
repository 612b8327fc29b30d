"""CPU oracle for the NVFP4 attention forward.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import
this module, and only as the checker or the timed CPU baseline; the product package never does.

What it restates (paths inside the reference project, graphcore-research/flash-attention):

* ``attention_ref``  -- flash_attn/cute/testing.py:323-434: fp32 ``softmax(scale * Q K^T + mask) V``
  with GQA by repeating kv heads (``:362-363``), bottom-right aligned causal mask
  (``construct_local_mask`` ``:249-288``: key j is masked when ``j > i + Sk - Sq``), rows that see
  no key give 0 (``:422-423``).  The LSE is ``logsumexp`` of the masked scaled scores, the pattern
  of tests/cute/test_flash_attn.py:1534-1539.
* the FLOP count ``flops`` -- flash_attn/cute/bench_utils.py:15-38.
* the quantised-path test hook of the reference (``q/k/v_descale`` multiply the inputs,
  ``intermediate_dtype`` rounds P before P.V; testing.py:353-360,429-431) is the model for
  ``attention_oracle_b``: dequantise with the scales, round P the way the kernel does, then P.V.

Parity status: the reference contains NO NVFP4 attention path (its forward asserts fp16/bf16
inputs, flash_attn/cute/interface.py:370), hence no golden vector pins FP4 results:
**NVFP4 parity is unpinned by the reference**.  What IS pinned, by fixtures generated from the
reference's own ``attention_ref`` (tests/golden/make_golden.py): ``attention_oracle_a`` on
dequantised inputs, including GQA, causal with Sq != Sk, and the LSE convention.

The NVFP4 number format restated here is the public one (OCP e2m1 elements, e4m3 scale per
16 elements, fp32 per-tensor scale) with the quantisation recipe stated for the benchmark
configurations: per-tensor scale = amax / (6 * 448); block scale = e4m3(block_amax / 6 /
per-tensor scale); elements = e2m1 round-to-nearest-even of x / (block scale * per-tensor scale).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# decision thresholds between neighbouring e2m1 magnitudes; a tie goes to the code with even
# mantissa bit (codes 0, 2, 4, 6), i.e. 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2,
# 3.5 -> 4, 5 -> 4
_E2M1_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
_E2M1_TIE_UP = np.array([False, True, False, True, False, True, False])  # tie rounds up?

LOG2_6 = math.log2(6.0)
P_SHIFT = 6          # constant up-shift of P in log2 units (kernel: kShift)
P_LAZY = 4           # lazy-rescale threshold in log2 units (kernel: kLazy)
P_EMIN = -6          # smallest block-scale exponent (kernel: kEMin; ue4m3 normals only)
BLOCK = 16


# --------------------------------------------------------------------------------------------
# number formats
# --------------------------------------------------------------------------------------------
def e2m1_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit e2m1 codes (sign in bit 3), round to nearest even, saturating at 6."""
    x = np.asarray(x, dtype=np.float32)
    mag = np.abs(x)
    code = np.zeros(x.shape, dtype=np.uint8)
    for i in range(7):
        up = (mag >= _E2M1_MID[i]) if _E2M1_TIE_UP[i] else (mag > _E2M1_MID[i])
        code += up.astype(np.uint8)
    sign = (np.signbit(x) & (code > 0)).astype(np.uint8)  # no negative zero needed
    return code | (sign << 3)


def e2m1_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    mag = E2M1_VALUES[code & 7]
    return np.where(code & 8, -mag, mag).astype(np.float32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """(..., n) 4-bit codes -> (..., n/2) bytes, even index in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = packed >> 4
    return out


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3 (fn: no inf, max 448) bytes, round to nearest even, saturating."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).clamp(-448.0, 448.0)
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(b, dtype=np.uint8)).view(torch.float8_e4m3fn)
    return t.to(torch.float32).numpy()


# --------------------------------------------------------------------------------------------
# NVFP4 quantiser (blocks of 16 along the LAST axis of x)
# --------------------------------------------------------------------------------------------
@dataclass
class NVFP4:
    data: np.ndarray      # uint8 (..., n/2) packed e2m1
    sf: np.ndarray        # uint8 (..., n/16) e4m3 block scales, linear layout
    scale: float          # fp32 per-tensor scale


def quantize_nvfp4(x: np.ndarray) -> NVFP4:
    x = np.asarray(x, dtype=np.float32)
    assert x.shape[-1] % BLOCK == 0
    amax = float(np.max(np.abs(x)))
    gs = np.float32(amax / (6.0 * 448.0)) if amax > 0 else np.float32(1.0)
    xb = x.reshape(x.shape[:-1] + (x.shape[-1] // BLOCK, BLOCK))
    bmax = np.max(np.abs(xb), axis=-1)
    sf_code = e4m3_encode(bmax / np.float32(6.0) / gs)
    sf = e4m3_decode(sf_code)
    denom = (sf * gs)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = np.where(denom > 0, xb / denom, 0.0).astype(np.float32)
    codes = e2m1_encode(scaled).reshape(x.shape)
    return NVFP4(pack_nibbles(codes), sf_code, float(gs))


def dequantize_nvfp4(q: NVFP4) -> np.ndarray:
    vals = e2m1_decode(unpack_nibbles(q.data))
    sf = e4m3_decode(q.sf)
    vb = vals.reshape(vals.shape[:-1] + (vals.shape[-1] // BLOCK, BLOCK))
    return (vb * (sf * np.float32(q.scale))[..., None]).reshape(vals.shape).astype(np.float32)


def sf_linear_to_tiled(sf: np.ndarray, col_tile_multiple: int = 1) -> np.ndarray:
    """(..., rows, cols) bytes -> (..., ceil(rows/128), CT, 512) bytes, CT = ceil(cols/4) rounded up
    to a multiple of col_tile_multiple; inside a tile the scale of (r, c) sits at
    (r % 32) * 16 + (r // 32) * 4 + c.  Zero padding."""
    rows, cols = sf.shape[-2:]
    rt = (rows + 127) // 128
    ct = ((cols + 3) // 4 + col_tile_multiple - 1) // col_tile_multiple * col_tile_multiple
    pad = np.zeros(sf.shape[:-2] + (rt * 128, ct * 4), dtype=np.uint8)
    pad[..., :rows, :cols] = sf
    t = pad.reshape(sf.shape[:-2] + (rt, 4, 32, ct, 4))        # (rt, r//32, r%32, ct, c)
    t = np.moveaxis(t, [-5, -2, -3, -4, -1], [-5, -4, -3, -2, -1])  # (rt, ct, r%32, r//32, c)
    return np.ascontiguousarray(t).reshape(sf.shape[:-2] + (rt, ct, 512))


# --------------------------------------------------------------------------------------------
# attention, oracle A: fp32 attention on (dequantised) inputs
# --------------------------------------------------------------------------------------------
def _causal_mask(sq: int, sk: int) -> torch.Tensor:
    i = torch.arange(sq)[:, None]
    j = torch.arange(sk)[None, :]
    return j > i + (sk - sq)


def _visibility_mask(sq: int, sk: int, causal: bool, window=(None, None)):
    """True where key j is MASKED for query i: the reference's construct_local_mask
    (flash_attn/cute/testing.py:249-288) with causal = right limit 0, bottom-right aligned.
    Returns None when nothing is masked."""
    left, right = window
    if causal:
        right = 0
    if left is None and right is None:
        return None
    i = torch.arange(sq)[:, None]
    j = torch.arange(sk)[None, :]
    m = torch.zeros(sq, sk, dtype=torch.bool)
    if right is not None:
        m |= j > i + (sk - sq) + right
    if left is not None:
        m |= j < i + (sk - sq) - left
    return m


def attention_oracle_a(q, k, v, causal=False, softmax_scale=None, window=(None, None), sink=None,
                       softcap: float = 0.0):
    """q (B,Sq,Hq,D), k (B,Sk,Hkv,D), v (B,Sk,Hkv,Dv) fp32 torch CPU tensors.
    softcap > 0: scores = softcap * tanh(scores / softcap) before masking (testing.py:373-374).
    Returns (out (B,Sq,Hq,Dv) fp32, lse (B,Hq,Sq) fp32)."""
    q, k, v = (torch.as_tensor(t, dtype=torch.float32) for t in (q, k, v))
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D)
    k = k.repeat_interleave(g, dim=2)
    v = v.repeat_interleave(g, dim=2)
    scores = torch.einsum("bthd,bshd->bhts", q * scale, k)
    if softcap and softcap > 0:
        scores = torch.tanh(scores / softcap) * softcap
    mask = _visibility_mask(Sq, Sk, causal, window)
    if mask is not None:
        scores = scores.masked_fill(mask, float("-inf"))
    if sink is not None:
        # one more logit per query head in the normaliser, no value row (testing.py:406-416)
        sk_ = torch.as_tensor(sink, dtype=torch.float32).reshape(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        ext = torch.cat([scores, sk_], dim=-1)
        lse = torch.logsumexp(ext, dim=-1)
        attn = torch.softmax(ext, dim=-1)[..., :-1]
    else:
        lse = torch.logsumexp(scores, dim=-1)
        attn = torch.softmax(scores, dim=-1)
    if mask is not None:
        attn = attn.masked_fill(torch.all(mask, dim=-1, keepdim=True), 0.0)
    attn = torch.nan_to_num(attn, nan=0.0)
    out = torch.einsum("bhts,bshd->bthd", attn, v)
    return out, lse


# --------------------------------------------------------------------------------------------
# attention, oracle B: the kernel's arithmetic model (P re-quantised to NVFP4)
# --------------------------------------------------------------------------------------------
# general ue4m3 block scales of the 64-key kernel (csrc/softmax.cuh, block_scales4_e4m3)
_POW2M1_C1, _POW2M1_C2 = np.float32(5.2904577), np.float32(2.6854515)
_LOG2_1P8 = torch.tensor([math.log2(1.0 + m / 8.0) for m in range(9)], dtype=torch.float32)


def quantize_p_block_model(x: torch.Tensor, m_ref: torch.Tensor, p_scale: str = "pow2"):
    """x: (..., 16 k) scaled scores in log2 units of ONE step of keys, m_ref: (..., 1) reference
    maximum in the same units (finite).  Returns (p_hat, p_sum): the de-quantised P' the tensor
    core multiplies with V, and the un-rounded row sums of P' (P' = 2^P_SHIFT * 2^(x - m_ref)).
    p_scale: "pow2" -- block scale 2^e, e = ceil(log2(block max / 6)); "e4m3" -- the smallest
    2^e (1 + m/8) >= block max / 6, found the way the kernel finds it (floor, a quadratic for
    8 (2^fr - 1), round to nearest of that + 0.5)."""
    xb = x.reshape(x.shape[:-1] + (x.shape[-1] // BLOCK, BLOCK))
    bmax = xb.amax(dim=-1, keepdim=True)
    t = bmax - m_ref[..., None] + P_SHIFT
    if p_scale == "e4m3":
        t = (t - np.float32(LOG2_6)).to(torch.float32)
        t = torch.where(torch.isfinite(t), torch.clamp(t, min=float(P_EMIN)), torch.full_like(t, float(P_EMIN)))
        e = torch.floor(t)
        fr = t - e
        g = fr * (fr * _POW2M1_C2 + _POW2M1_C1)
        m = torch.round(g + np.float32(0.4999995))            # round half to even, like the magic add
        lm = _LOG2_1P8[m.long()]
        scale = torch.exp2(e) * (1.0 + m / 8.0)
        p_scaled = torch.exp2(xb - (m_ref[..., None] - P_SHIFT) - e - lm)
        codes = e2m1_encode(p_scaled.numpy())
        p_hat = torch.from_numpy(e2m1_decode(codes)) * scale
        p_sum = (p_scaled.sum(dim=-1) * scale[..., 0]).sum(dim=-1)
        return p_hat.reshape(x.shape), p_sum
    e = torch.clamp(torch.ceil(t - LOG2_6), float(P_EMIN), 8.0)
    e = torch.where(torch.isfinite(t), e, torch.full_like(e, float(P_EMIN)))
    p_scaled = torch.exp2(xb - (m_ref[..., None] - P_SHIFT + e))          # in [0, 6]
    codes = e2m1_encode(p_scaled.numpy())
    p_hat = torch.from_numpy(e2m1_decode(codes)) * torch.exp2(e)
    p_sum = (p_scaled.sum(dim=-1) * torch.exp2(e[..., 0])).sum(dim=-1)
    return p_hat.reshape(x.shape), p_sum


def attention_oracle_b(qd, kd, vd, sl2: float, v_scale_out: float = 1.0, causal=False,
                       num_splits: int = 1, window=(None, None), sink=None,
                       step_keys: int = 128, ascending: bool = False, softcap_c1: float = 0.0,
                       p_scale: str = "pow2"):
    """Kernel model.  qd (B,Sq,Hq,D), kd (B,Sk,Hkv,D), vd (B,Sk,Hkv,Dv): fp32 values the tensor
    core sees (e2m1 * block scale, WITHOUT the per-tensor scales); sl2 = softmax_scale * q_scale
    * k_scale * log2(e); v_scale_out = v_scale.  Walks the K/V blocks of 128 keys from the last
    visible one to the first with the lazy reference maximum, like the kernel.
    num_splits > 1 models the split-KV path: the visited blocks of a tile are cut into
    num_splits contiguous shares (ceil division, in visit order), each share starts from a fresh
    reference maximum, and the shares are merged with exp(lse_i - lse) weights (the combine
    step of the reference, tests/cute/test_flash_attn_fast.py:295-300).
    step_keys / ascending select the kernel that is modelled: the 128-key kernel takes steps of
    128 keys from the last visible block down (the defaults); the 64-key kernel
    (csrc/attn_ws64.cuh) takes steps of 64 keys upwards from key 0.  The set of visited keys is
    the same (whole 128-key blocks); the step decides where the lazy reference maximum may move,
    hence the scaling under which P is rounded to e2m1.
    softcap_c1 > 0 models the soft cap: the raw scores become tanh(raw * softcap_c1) with
    softcap_c1 = softmax_scale * q_scale * k_scale / softcap, and the caller passes
    sl2 = softcap * log2(e): everything after that is unchanged.
    p_scale selects the rule of the P block scales (see quantize_p_block_model).
    Returns (out fp32 (B,Sq,Hq,Dv) before bf16 rounding, lse (B,Hq,Sq))."""
    assert step_keys in (64, 128) and (step_keys == 128 or num_splits == 1)
    sub = 128 // step_keys
    qd, kd, vd = (torch.as_tensor(t, dtype=torch.float32) for t in (qd, kd, vd))
    B, Sq, Hq, D = qd.shape
    Sk, Hkv, Dv = kd.shape[1], kd.shape[2], vd.shape[3]
    g = Hq // Hkv
    out = torch.zeros(B, Sq, Hq, Dv)
    lse = torch.full((B, Hq, Sq), float("-inf"))
    for b in range(B):
        for h in range(Hq):
            hk = h // g
            for m0 in range(0, Sq, 128):
                rows = slice(m0, min(m0 + 128, Sq))
                nr = rows.stop - rows.start
                n_blocks = (Sk + 127) // 128
                s_all = torch.full((nr, n_blocks * 128), float("-inf"))   # keys >= Sk never count
                s_all[:, :Sk] = (qd[b, rows, h] @ kd[b, :, hk].T)         # raw scores
                if softcap_c1 > 0:
                    s_all[:, :Sk] = torch.tanh(s_all[:, :Sk] * softcap_c1)
                v_pad = torch.zeros(n_blocks * 128, Dv)
                v_pad[:Sk] = vd[b, :, hk]
                left, right = window
                if causal:
                    right = 0
                n_min = 0
                if right is not None:
                    last = m0 + 128 + Sk - Sq + right
                    n_blocks = min(n_blocks, max(0, (last + 127) // 128))
                if left is not None:
                    first = m0 + Sk - Sq - left
                    n_min = min(n_blocks, max(0, first // 128))
                mask = _visibility_mask(Sq, Sk, causal, window)
                if mask is not None:
                    s_all[:, :Sk] = s_all[:, :Sk].masked_fill(mask[rows], float("-inf"))
                if ascending:
                    # a tile that is cut on the left visits the two blocks of the window's left
                    # edge last (csrc/attn_ws64.cuh, window_visit_block)
                    blocks = list(range(n_min, n_blocks))
                    if left is not None and len(blocks) > 2 and (m0 + Sk - Sq - left) > 0:
                        blocks = blocks[2:] + blocks[:2]
                    visit = [nb * sub + h for nb in blocks for h in range(sub)]
                else:
                    visit = [nb * sub + h for nb in range(n_blocks - 1, n_min - 1, -1)
                             for h in range(sub - 1, -1, -1)]
                per = (len(visit) + num_splits - 1) // num_splits if visit else 0
                parts = []
                for sp in range(num_splits):
                    share = visit[sp * per:(sp + 1) * per] if per else []
                    m_ref = torch.full((nr,), float("-inf"))
                    l_sum = torch.zeros(nr)
                    acc = torch.zeros(nr, Dv)
                    for nb in share:
                        s = s_all[:, nb * step_keys:(nb + 1) * step_keys]
                        m_loc = s.amax(dim=-1)
                        keep = torch.isfinite(m_ref) & ((m_loc - m_ref) * sl2 <= P_LAZY)
                        m_new = torch.where(keep, m_ref, torch.maximum(m_ref, m_loc))
                        f = torch.where(torch.isfinite(m_ref), torch.exp2((m_ref - m_new) * sl2),
                                        torch.zeros(nr))
                        f = torch.nan_to_num(f, nan=0.0)
                        acc = acc * f[:, None]
                        l_sum = l_sum * f
                        m_ref = m_new
                        msc = torch.where(torch.isfinite(m_ref), m_ref * sl2, torch.zeros(nr))
                        p_hat, p_sum = quantize_p_block_model(s * sl2, msc[:, None], p_scale)
                        acc = acc + p_hat @ v_pad[nb * step_keys:(nb + 1) * step_keys]
                        l_sum = l_sum + p_sum
                    if sink is not None and sp == 0:
                        # the sink joins the row sum of split 0; a row without keys keeps LSE = sink
                        sv = float(sink[h])
                        has = torch.isfinite(m_ref)
                        l_sum = torch.where(has, l_sum + torch.exp2(P_SHIFT + sv * math.log2(math.e) - m_ref * sl2),
                                            l_sum)
                    ok = l_sum > 0
                    safe = torch.where(ok, l_sum, torch.ones(nr))
                    o_part = torch.where(ok[:, None], acc * (v_scale_out / safe)[:, None],
                                         torch.zeros(nr, Dv))
                    l_part = torch.where(
                        ok, (m_ref * sl2 + torch.log2(safe) - P_SHIFT) * math.log(2.0),
                        torch.full((nr,), float("-inf")))
                    if sink is not None and sp == 0:
                        l_part = torch.where(torch.isfinite(m_ref), l_part, torch.full((nr,), float(sink[h])))
                    parts.append((o_part, l_part))
                if num_splits == 1:
                    out[b, rows, h], lse[b, h, rows] = parts[0]
                else:
                    l_all = torch.stack([lp for _, lp in parts])                # (splits, nr)
                    m = l_all.amax(dim=0)
                    fin = torch.isfinite(m)
                    w = torch.where(fin[None], torch.exp(l_all - torch.where(fin, m, torch.zeros(nr))[None]),
                                    torch.zeros_like(l_all))
                    tot = torch.where(fin, w.sum(dim=0), torch.ones(nr))
                    o = sum(w[i][:, None] * parts[i][0] for i in range(num_splits))
                    out[b, rows, h] = torch.where(fin[:, None], o / tot[:, None], torch.zeros(nr, Dv))
                    lse[b, h, rows] = torch.where(fin, m + torch.log(tot), torch.full((nr,), float("-inf")))
    return out, lse


# --------------------------------------------------------------------------------------------
# accounting
# --------------------------------------------------------------------------------------------
def attention_flops(B, Sq, Sk, Hq, D, Dv, causal):
    """FLOPs of one forward, formula of flash_attn/cute/bench_utils.py:15-38."""
    avg_sk = (max(0, Sk - Sq) + Sk) / 2 if causal else Sk
    return B * Hq * 2 * Sq * avg_sk * (D + Dv)


def error_metrics(x: torch.Tensor, ref: torch.Tensor):
    x, ref = x.float(), ref.float()
    finite = torch.isfinite(ref)
    d = torch.where(finite, x - ref, torch.zeros_like(ref))
    r = torch.where(finite, ref, torch.zeros_like(ref))
    return {"max_abs": float(d.abs().max()),
            "rel_rms": float(d.norm() / max(float(r.norm()), 1e-30))}
