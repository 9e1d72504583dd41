"""Plain PyTorch statements of every operator, with fp32 math.

These are (a) the CPU execution path (gloo tests, meta/CPU debugging) and
(b) the oracles the CUDA kernels are tested against.  They restate the
reference's math: RMSNorm (torchtitan/models/common/nn_modules.py:133-147),
RoPE (models/common/rope.py:253-346), SwiGLU (models/common/feed_forward.py:53),
cross entropy with sum reduction (components/loss.py:27-62), AdamW
(torch.optim.AdamW semantics, components/optimizer/optimizer.py:378-399) and the
token-choice router (models/common/moe.py:277-335).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


# ---------------------------------------------------------------- RMSNorm
def rms_norm_fwd(x: torch.Tensor, weight: torch.Tensor | None, eps: float):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = xf * rstd
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype), rstd.squeeze(-1)


def rms_norm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor | None, rstd: torch.Tensor):
    xf, dyf = x.float(), dy.float()
    r = rstd.float().unsqueeze(-1)
    xhat = xf * r
    wdy = dyf * weight.float() if weight is not None else dyf
    c = (wdy * xhat).mean(dim=-1, keepdim=True)
    dx = (wdy - xhat * c) * r
    dw = None
    if weight is not None:
        dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(dim=0)
    return dx.to(x.dtype), dw


# ------------------------------------------------------------------- RoPE
def rope_table(head_dim: int, max_pos: int, theta: float, scaling: str = "none", *, scaling_factor: float = 8.0,
               low_freq_factor: float = 1.0, high_freq_factor: float = 4.0, original_max_pos: int = 8192,
               rope_factor: float = 1.0, beta_fast: float = 32.0, beta_slow: float = 1.0,
               original_seq_len: int = 4096, truncate: bool = True) -> torch.Tensor:
    """``[max_pos, head_dim]`` fp32 table holding ``cos | sin`` of ``pos * inv_freq``."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[:half].float() / head_dim))
    if scaling == "llama":
        wavelen = 2 * math.pi / inv
        low_wl = original_max_pos / low_freq_factor
        high_wl = original_max_pos / high_freq_factor
        scaled = torch.where(wavelen > low_wl, inv / scaling_factor, inv)
        s = (original_max_pos / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
        smooth = (1 - s) * inv / scaling_factor + s * inv
        medium = (~(wavelen < high_wl)) & (~(wavelen > low_wl))
        inv = torch.where(medium, smooth, scaled)
    elif scaling == "yarn" and rope_factor > 1.0:
        inv = yarn_inv_freq(head_dim, theta, rope_factor, beta_fast, beta_slow, original_seq_len, truncate)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv.float())
    return torch.cat([ang.cos(), ang.sin()], dim=-1).contiguous()


def yarn_inv_freq(dim, base, factor, beta_fast, beta_slow, original_seq_len, truncate=True):
    def corr_dim(n_rot):
        return dim * math.log(original_seq_len / (n_rot * 2 * math.pi)) / (2 * math.log(base))

    low, high = corr_dim(beta_fast), corr_dim(beta_slow)
    if truncate:
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    smooth = 1 - ramp
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    return inv / factor * (1 - smooth) + inv * smooth


def rope_apply(x: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, interleaved: bool,
               inverse: bool = False) -> torch.Tensor:
    """Rotate ``x[T, H, D]`` by the angles of ``positions[T]``.

    ``interleaved`` pairs dims ``(2i, 2i+1)`` (Llama "complex" RoPE); otherwise
    dims ``(i, i + D/2)`` (rotate-half).  ``inverse`` applies the transpose
    rotation, i.e. the backward pass.  ``table`` may be narrower than ``D``
    (partial rotary): only the first ``table.shape[1]`` dims rotate.
    """
    rot = table.shape[1]
    half = rot // 2
    cs = table[positions.long()]
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    if inverse:
        sin = -sin
    xf = x.float()
    xr, xpass = xf[..., :rot], xf[..., rot:]
    if interleaved:
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
        o0 = x0 * cos - x1 * sin
        o1 = x0 * sin + x1 * cos
        out = torch.stack([o0, o1], dim=-1).flatten(-2)
    else:
        x0, x1 = xr[..., :half], xr[..., half:]
        out = torch.cat([x0 * cos - x1 * sin, x1 * cos + x0 * sin], dim=-1)
    if xpass.shape[-1]:
        out = torch.cat([out, xpass], dim=-1)
    return out.to(x.dtype)


# ----------------------------------------------------------------- SwiGLU
def swiglu_fwd(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def swiglu_bwd(gate: torch.Tensor, up: torch.Tensor, dout: torch.Tensor):
    g, u, d = gate.float(), up.float(), dout.float()
    sig = torch.sigmoid(g)
    silu = g * sig
    dg = d * u * (sig + silu * (1 - sig))
    du = d * silu
    return dg.to(gate.dtype), du.to(up.dtype)


# ---------------------------------------------------------- cross entropy
def cross_entropy_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, grad_scale: torch.Tensor | float):
    """Sum-reduced CE and ``dlogits = (softmax - onehot) * grad_scale``.

    Returns ``(loss_sum fp32 scalar, dlogits in logits.dtype, n_valid)``.
    """
    lf = logits.float()
    valid = labels != IGNORE_INDEX
    lse = torch.logsumexp(lf, dim=-1)
    safe = labels.clamp_min(0).long()
    tgt = lf.gather(-1, safe[:, None]).squeeze(-1)
    loss = ((lse - tgt) * valid).sum()
    p = torch.exp(lf - lse[:, None])
    p.scatter_add_(-1, safe[:, None], -torch.ones_like(tgt)[:, None])
    p = p * valid[:, None]
    if isinstance(grad_scale, torch.Tensor):
        grad_scale = grad_scale.float()
    return loss, (p * grad_scale).to(logits.dtype), valid.sum()


# ------------------------------------------------------------------ AdamW
def adamw_step(master: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
               *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               grad_scale: torch.Tensor | float = 1.0, out_lowp: torch.Tensor | None = None) -> None:
    """In-place decoupled-weight-decay Adam on flat fp32 ``master``.

    ``exp_avg``/``exp_avg_sq`` may be bf16 (math is fp32, state is rounded on
    store).  ``grad_scale`` is the clip coefficient; ``out_lowp`` receives the
    updated parameters cast to its dtype.
    """
    g = grad.float() * grad_scale
    m = exp_avg.float().mul_(beta1).add_(g, alpha=1 - beta1)
    v = exp_avg_sq.float().mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    master.mul_(1 - lr * weight_decay)
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    master.addcdiv_(m, denom, value=-lr / bc1)
    exp_avg.copy_(m)
    exp_avg_sq.copy_(v)
    if out_lowp is not None:
        out_lowp.copy_(master)


# -------------------------------------------------------------- attention
def _block_mask(Tq: int, Tk: int, device, causal: bool, causal_offset: int, kv_first, window: int) -> torch.Tensor:
    """The flash kernels' mask in local indices: row i sees keys max(kv_first[i], i + offset - window + 1) <= j <= i + offset."""
    rows = torch.arange(Tq, device=device)[:, None]
    cols = torch.arange(Tk, device=device)[None, :]
    mask = torch.ones(Tq, Tk, dtype=torch.bool, device=device)
    if causal:
        mask &= cols <= rows + causal_offset
    if kv_first is not None:
        mask &= cols >= kv_first.long()[:, None]
    if window:
        mask &= cols > rows + causal_offset - window
    return mask


def block_attention_fwd(q, k, v, scale: float, causal: bool = True, causal_offset: int = 0, kv_first=None, window: int = 0):
    """Dense-math counterpart of ``flash_fwd``: ``(o [Tq, Hq, D] in q's dtype, lse [Hq, Tq] fp32)``; rows that see no
    key get ``o = 0`` and ``lse = -inf``."""
    Tq, Hq, _ = q.shape
    Tk, Hkv, _ = k.shape
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    mask = _block_mask(Tq, Tk, q.device, causal, causal_offset, kv_first, window)
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.where(mask[None], torch.exp(s - safe[..., None]), torch.zeros_like(s))
    return torch.matmul(p, vf).transpose(0, 1).to(q.dtype), lse


def block_attention_bwd(d_o, q, k, v, o, lse, scale: float, causal: bool = True, causal_offset: int = 0, kv_first=None,
                        window: int = 0):
    """Dense-math counterpart of ``flash_bwd``.  ``o`` and ``lse`` may be the *merged* result over several key
    blocks: with ``P = exp(s - lse)`` and ``delta = rowsum(dO * O)`` the returned ``dq`` is this block's share
    and ``dk`` / ``dv`` are exact for this block's keys."""
    Tq, Hq, _ = q.shape
    Tk, Hkv, _ = k.shape
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    dof = d_o.float().transpose(0, 1)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    mask = _block_mask(Tq, Tk, q.device, causal, causal_offset, kv_first, window)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.where(mask[None], torch.exp(s - safe[..., None]), torch.zeros_like(s))
    delta = (d_o.float() * o.float()).sum(-1).transpose(0, 1)              # [Hq, Tq]
    dp = torch.matmul(dof, vf.transpose(1, 2))
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.matmul(ds, kf).transpose(0, 1)
    dk = torch.matmul(ds.transpose(1, 2), qf).view(Hkv, rep, Tk, -1).sum(1).transpose(0, 1)
    dv = torch.matmul(p.transpose(1, 2), dof).view(Hkv, rep, Tk, -1).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def attention_merge_(acc_o: torch.Tensor, acc_lse: torch.Tensor, o: torch.Tensor, lse: torch.Tensor) -> None:
    """In place: fold one block's normalised output ``o [T, H, D]`` / ``lse [H, T]`` into the fp32 running pair."""
    new = torch.logaddexp(acc_lse, lse)
    safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
    wa = torch.where(torch.isinf(acc_lse), torch.zeros_like(new), torch.exp(acc_lse - safe)).transpose(0, 1)[..., None]
    wb = torch.where(torch.isinf(lse), torch.zeros_like(new), torch.exp(lse - safe)).transpose(0, 1)[..., None]
    acc_o.mul_(wa).add_(o.float() * wb)
    acc_lse.copy_(new)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float, causal: bool = True,
                  doc_ids: torch.Tensor | None = None, window: int | None = None,
                  q_pos: torch.Tensor | None = None, k_pos: torch.Tensor | None = None,
                  sinks: torch.Tensor | None = None):
    """Dense-math attention over folded tokens.

    ``q[Tq, Hq, D]``, ``k/v[Tk, Hkv, D(v)]``; GQA by head repetition.  ``doc_ids``
    (``[T]`` ints, same for q and k unless a tuple ``(q_doc, k_doc)``) restricts
    attention to the same document; ``q_pos``/``k_pos`` are global token indices
    used by the causal and sliding-window tests (default ``arange``).  ``sinks``
    (``[Hq]``) adds a per-head logit to the softmax denominator.
    Returns ``(out[Tq, Hq, Dv], lse[Hq, Tq])``.
    """
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    rep = Hq // Hkv
    qf = q.float().transpose(0, 1)  # [Hq, Tq, D]
    kf = k.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale  # [Hq, Tq, Tk]
    dev = q.device
    qp = torch.arange(Tq, device=dev) if q_pos is None else q_pos
    kp = torch.arange(Tk, device=dev) if k_pos is None else k_pos
    mask = torch.ones(Tq, Tk, dtype=torch.bool, device=dev)
    if causal:
        mask &= qp[:, None] >= kp[None, :]
    if window is not None and window > 0:
        mask &= (qp[:, None] - kp[None, :]) < window
    if doc_ids is not None:
        qd, kd = doc_ids if isinstance(doc_ids, tuple) else (doc_ids, doc_ids)
        mask &= qd[:, None] == kd[None, :]
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s_ext = torch.cat([s, sinks.float()[:, None, None].expand(Hq, Tq, 1)], dim=-1)
        lse = torch.logsumexp(s_ext, dim=-1)
    else:
        lse = torch.logsumexp(s, dim=-1)
    lse_safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - lse_safe[..., None])
    p = torch.where(mask[None], p, torch.zeros_like(p))
    out = torch.matmul(p, vf).transpose(0, 1)
    return out.to(q.dtype), lse


# ----------------------------------------------------------------- router
def router_topk(scores_logits: torch.Tensor, top_k: int, score_func: str, expert_bias: torch.Tensor | None,
                route_norm: bool, route_scale: float, num_expert_groups: int | None = None,
                num_limited_groups: int | None = None):
    """Token-choice routing on fp32 gate logits ``[T, E]``.

    Returns ``(top_scores[T,K] fp32, selected[T,K] int64, tokens_per_expert[E] fp32)``.
    """
    logits = scores_logits.float()
    scores = torch.softmax(logits, dim=-1) if score_func == "softmax" else torch.sigmoid(logits)
    sel_scores = scores if expert_bias is None else scores + expert_bias.float()
    E = scores.shape[-1]
    if num_expert_groups and num_limited_groups and num_expert_groups > 1:
        T = scores.shape[0]
        grp = sel_scores.view(T, num_expert_groups, E // num_expert_groups)
        gscore = grp.topk(2, dim=-1).values.sum(dim=-1)
        keep = gscore.topk(num_limited_groups, dim=-1).indices
        gmask = torch.zeros(T, num_expert_groups, dtype=torch.bool, device=scores.device)
        gmask.scatter_(1, keep, True)
        sel_scores = grp.masked_fill(~gmask[..., None], float("-inf")).reshape(T, E)
    sel = sel_scores.topk(top_k, dim=-1, sorted=False).indices
    top = scores.gather(-1, sel)
    if route_norm:
        top = top / (top.sum(dim=-1, keepdim=True) + 1e-20)
    top = top * route_scale
    counts = torch.zeros(E, dtype=torch.float32, device=scores.device)
    counts.scatter_add_(0, sel.reshape(-1), torch.ones(sel.numel(), dtype=torch.float32, device=scores.device))
    return top, sel, counts


# ---------------------------------------------------------------------------------------------
# fp8 quantisation (oracles of ops/csrc/quant.cu)
# ---------------------------------------------------------------------------------------------
def mxfp8_scale_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Unbiased exponent ``e`` of the smallest power of two ``2^e >= amax / 448`` (RCEIL), clamped to
    the e8m0 range; zero blocks get the smallest scale."""
    m, ex = torch.frexp(amax.float() / 448.0)      # amax / 448 = m * 2^ex, m in [0.5, 1)
    e = torch.where(m == 0.5, ex - 1, ex).clamp(-126, 127)
    return torch.where(amax > 0, e, torch.full_like(e, -127))


def mxfp8_fake_quant(x: torch.Tensor, axis: int) -> torch.Tensor:
    """MXFP8 round trip of ``x[R, C]`` with 1x32 blocks along ``axis`` (ragged last block allowed on axis 0)."""
    xt = x.float() if axis == 1 else x.float().t()
    R, C = xt.shape
    pad = (-C) % 32
    if pad:
        xt = torch.nn.functional.pad(xt, (0, pad))
    blocks = xt.reshape(R, -1, 32)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    e = mxfp8_scale_exponent(amax)
    scale = torch.exp2(e.float())
    q = (blocks / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale
    out = q.reshape(R, -1)[:, :C]
    out = out if axis == 1 else out.t()
    return out.to(x.dtype)


def float8_pow2_exponents(amax: torch.Tensor) -> torch.Tensor:
    """e8m0 byte of the smallest power of two >= amax / 448 (uint8; 1 for an all-zero row)."""
    v = (amax.float() / 448.0).clamp_min(2.0 ** -126)
    m, e = torch.frexp(v)                          # v = m * 2^e, m in [0.5, 1)
    e = torch.where(m == 0.5, e - 1, e)            # exact powers of two keep their exponent
    return (e + 127).clamp(1, 254).to(torch.uint8)


def float8_rowwise_fake_quant(x: torch.Tensor, pow2: bool = True) -> torch.Tensor:
    """Row-wise float8 (e4m3) round trip.  ``pow2`` rounds each row's scale up to a power of two, the default of the
    reference's row-wise recipe (torchao ``round_scales_to_power_of_2``); it makes the scaled values exactly
    representable products, which is what lets the GEMM run on the block-scaled tensor-core kernel."""
    xf = x.float()
    amax = xf.abs().amax(dim=1, keepdim=True)
    if pow2:
        scale = torch.exp2(float8_pow2_exponents(amax).float() - 127.0)
    else:
        scale = amax.clamp_min(1e-12) / 448.0
    return ((xf / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale).to(x.dtype)
