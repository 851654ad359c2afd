"""Training-side kernel wrappers (csrc/train_sm100.cu) with PyTorch reference twins."""

from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import check_rc, ptr, stream_handle

c_int, c_ll, c_float, c_vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _lib() -> ctypes.CDLL:
    lib = _native.load("rb_train")
    if not getattr(lib, "_rb_typed", False):
        lib.rb_logprob_entropy_fwd.argtypes = [c_vp, c_ll, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp]
        lib.rb_logprob_entropy_bwd.argtypes = [c_vp, c_ll, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_vp]
        lib.rb_rmsnorm_bwd.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_int, c_float, c_vp]
        lib.rb_rope.argtypes = [c_vp, c_vp, c_vp, c_vp, c_ll, c_int, c_int, c_ll, c_ll, c_int, c_int, c_vp]
        lib.rb_sumsq_partial.argtypes = [c_vp, c_ll, c_int, c_float, c_vp, c_vp]
        lib.rb_adamw.argtypes = [c_vp, c_vp, c_vp, c_vp, c_int, c_vp, c_ll, c_float, c_float, c_float, c_float, c_float,
                                 c_int, c_float, c_vp, c_vp]
        lib.rb_accumulate_f32_bf16.argtypes = [c_vp, c_vp, c_ll, c_vp]
        for f in ("rb_logprob_entropy_fwd", "rb_logprob_entropy_bwd", "rb_rmsnorm_bwd", "rb_rope", "rb_sumsq_partial",
                  "rb_adamw", "rb_accumulate_f32_bf16", "rb_rmsnorm_bwd_num_partials", "rb_sumsq_num_partials"):
            getattr(lib, f).restype = c_int
        lib._rb_typed = True
    return lib


# ---------------------------------------------------------------- log-prob / entropy from logits
def logprob_entropy_reference(logits: torch.Tensor, targets: torch.Tensor, need_entropy: bool = True):
    lp_all = torch.log_softmax(logits.float(), -1)
    lse = torch.logsumexp(logits.float(), -1)
    safe = targets.long().clamp(min=0)
    lp = lp_all.gather(-1, safe[:, None]).squeeze(-1)
    lp = torch.where(targets >= 0, lp, torch.zeros_like(lp))
    ent = -(lp_all.exp() * lp_all).sum(-1) if need_entropy else None
    return lp, lse, ent


def logprob_entropy_fwd(logits: torch.Tensor, targets: torch.Tensor, need_entropy: bool = True):
    """Per-row ``log p(target)``, log-sum-exp and entropy from fp32 logits ``[R, V]``."""
    if not logits.is_cuda:
        return logprob_entropy_reference(logits, targets, need_entropy)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and targets.dtype == torch.int32
    R, V = logits.shape
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    lse = torch.empty_like(lp)
    ent = torch.empty_like(lp) if need_entropy else None
    rc = _lib().rb_logprob_entropy_fwd(ptr(logits), logits.stride(0), R, V, ptr(targets), ptr(lp), ptr(lse), ptr(ent),
                                       stream_handle(logits.device))
    check_rc(rc, "rb_logprob_entropy_fwd")
    return lp, lse, ent


def logprob_entropy_bwd(logits, targets, lse, entropy, g_logprob, g_entropy, out: torch.Tensor | None = None):
    """``dlogits`` (bf16) for upstream gradients of the per-row log-prob and entropy."""
    if not logits.is_cuda:
        lp_all = logits.float() - lse[:, None]
        p = lp_all.exp()
        onehot = torch.zeros_like(p)
        valid = targets >= 0
        onehot[valid, targets[valid].long()] = 1.0
        d = (g_logprob * valid)[:, None] * (onehot - p)
        if g_entropy is not None:
            d = d - g_entropy[:, None] * p * (lp_all + entropy[:, None])
        return d
    R, V = logits.shape
    if out is None:
        out = torch.empty(R, V, dtype=torch.bfloat16, device=logits.device)
    rc = _lib().rb_logprob_entropy_bwd(ptr(logits), logits.stride(0), R, V, ptr(targets), ptr(lse), ptr(entropy),
                                       ptr(g_logprob), ptr(g_entropy), ptr(out), out.stride(0), stream_handle(logits.device))
    check_rc(rc, "rb_logprob_entropy_bwd")
    return out


# ---------------------------------------------------------------- RMSNorm backward
def rmsnorm_bwd(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, eps: float):
    """Returns ``(dx, dw)`` with dw in fp32."""
    if not x.is_cuda:
        xf = x.float().detach().requires_grad_(True)
        wf = w.float().detach().requires_grad_(True)
        y = wf * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps))
        y.backward(dy.float())
        return xf.grad.to(x.dtype), wf.grad
    d = x.shape[-1]
    x2, dy2 = x.reshape(-1, d), dy.reshape(-1, d)
    assert x2.is_contiguous() and dy2.is_contiguous() and d * 4 <= 48 * 1024
    dx = torch.empty_like(x2)
    nparts = _lib().rb_rmsnorm_bwd_num_partials()
    part = torch.empty(nparts, d, dtype=torch.float32, device=x.device)
    rc = _lib().rb_rmsnorm_bwd(ptr(x2), ptr(w), ptr(dy2), ptr(dx), ptr(part), x2.shape[0], d, eps, stream_handle(x.device))
    check_rc(rc, "rb_rmsnorm_bwd")
    return dx.reshape(x.shape), part.sum(0)


# ---------------------------------------------------------------- RoPE (training, no cache)
def rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, backward: bool = False,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate ``x [T, H, D]`` (heads packed, any row stride) by +angle (forward) or -angle (backward); ``out`` may be
    a ``[T, H, D]`` view with its own row stride (e.g. the q columns of a fused QKV gradient)."""
    T, H, D = x.shape
    if not x.is_cuda:
        cs = table[positions.long()]
        c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
        if backward:
            s = -s
        lo, hi = x[..., : D // 2].float(), x[..., D // 2:].float()
        res = torch.cat([lo * c - hi * s, hi * c + lo * s], -1).to(x.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert x.stride(2) == 1 and x.stride(1) == D and positions.dtype == torch.int32
    y = torch.empty(T, H, D, dtype=x.dtype, device=x.device) if out is None else out
    assert y.shape == x.shape and y.stride(2) == 1 and y.stride(1) == D
    rc = _lib().rb_rope(ptr(x), ptr(y), ptr(positions), ptr(table), T, H, D, x.stride(0), y.stride(0), table.shape[0],
                        int(backward), stream_handle(x.device))
    check_rc(rc, "rb_rope")
    return y


# ---------------------------------------------------------------- optimizer pieces
def sumsq(g: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Sum of squares of ``g * scale`` as a device scalar (fp32)."""
    if not g.is_cuda:
        return (g.float() * scale).pow(2).sum()
    n = _lib().rb_sumsq_num_partials()
    part = torch.empty(n, dtype=torch.float32, device=g.device)
    rc = _lib().rb_sumsq_partial(ptr(g), g.numel(), int(g.dtype == torch.float32), scale, ptr(part), stream_handle(g.device))
    check_rc(rc, "rb_sumsq_partial")
    return part.sum()


def adamw_step(master, exp_avg, exp_avg_sq, grad, param_bf16, lr, beta1, beta2, eps, weight_decay, step,
               grad_scale: float = 1.0, clip_coef: torch.Tensor | None = None) -> None:
    """Fused AdamW on flat tensors: fp32 master + moments, bf16/fp32 grads, bf16 write-back."""
    if not master.is_cuda:
        g = grad.float() * grad_scale
        if clip_coef is not None:
            g = g * float(clip_coef)
        exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        master.mul_(1 - lr * weight_decay)
        master.addcdiv_(exp_avg / bc1, (exp_avg_sq / bc2).sqrt() + eps, value=-lr)
        if param_bf16 is not None:
            param_bf16.copy_(master.to(param_bf16.dtype))
        return
    rc = _lib().rb_adamw(ptr(master), ptr(exp_avg), ptr(exp_avg_sq), ptr(grad), int(grad.dtype == torch.float32),
                         ptr(param_bf16), master.numel(), lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                         ptr(clip_coef), stream_handle(master.device))
    check_rc(rc, "rb_adamw")


# ------------------------------------------------------------------------------ small activation kernels
def _unary(x: torch.Tensor, dy: torch.Tensor | None, mode: int, cap: float) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
    out = torch.empty_like(x)
    lib = _lib()
    lib.rb_unary.argtypes = [c_vp, c_vp, c_vp, c_ll, c_int, c_float, c_vp]
    rc = lib.rb_unary(ptr(x), ptr(dy.contiguous()) if dy is not None else None, ptr(out), x.numel(), mode, cap, stream_handle(x.device))
    check_rc(rc, "rb_unary")
    return out


def relu2(x: torch.Tensor) -> torch.Tensor:
    """``relu(x)**2`` (the MLP activation of dev/speedrun/single-file.py:973-975)."""
    return _unary(x, None, 0, 1.0) if x.is_cuda else torch.relu(x.float()).square().to(x.dtype)


def relu2_backward(x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    return _unary(x, dy, 0, 1.0) if x.is_cuda else (2 * torch.relu(x.float()) * dy.float()).to(x.dtype)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(x / cap)`` (logit soft-capping, dev/speedrun/single-file.py:1140)."""
    return _unary(x, None, 1, cap) if x.is_cuda else (cap * torch.tanh(x.float() / cap)).to(x.dtype)


def softcap_backward(x: torch.Tensor, dy: torch.Tensor, cap: float) -> torch.Tensor:
    return _unary(x, dy, 1, cap) if x.is_cuda else ((1 - torch.tanh(x.float() / cap) ** 2) * dy.float()).to(x.dtype)


def log_softmax(x: torch.Tensor) -> torch.Tensor:
    """Row log-softmax of fp32 ``[rows, cols]``."""
    if not x.is_cuda:
        return torch.log_softmax(x.float(), -1)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    out = torch.empty_like(x)
    lib = _lib()
    lib.rb_log_softmax.argtypes = [c_vp, c_vp, c_vp, c_int, c_int, c_vp]
    check_rc(lib.rb_log_softmax(ptr(x), None, ptr(out), x.shape[0], x.shape[1], stream_handle(x.device)), "rb_log_softmax")
    return out


def log_softmax_backward(y: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """Gradient w.r.t. the input given the forward output ``y`` and ``dy``."""
    if not y.is_cuda:
        return dy.float() - torch.exp(y.float()) * dy.float().sum(-1, keepdim=True)
    out = torch.empty_like(y)
    lib = _lib()
    lib.rb_log_softmax.argtypes = [c_vp, c_vp, c_vp, c_int, c_int, c_vp]
    check_rc(lib.rb_log_softmax(ptr(y), ptr(dy.contiguous()), ptr(out), y.shape[0], y.shape[1], stream_handle(y.device)), "rb_log_softmax(bwd)")
    return out


# ---------------------------------------------------------------- pooling / vector add (small kernels of the dev tree)
def adaptive_avg_pool2d(x: torch.Tensor, output_size: tuple[int, int]) -> torch.Tensor:
    """``[N, C, H, W]`` fp32 -> ``[N, C, OH, OW]`` (windows as in ``torch.nn.functional.adaptive_avg_pool2d``)."""
    if not x.is_cuda:
        return torch.nn.functional.adaptive_avg_pool2d(x, output_size)
    assert x.dtype == torch.float32 and x.dim() == 4
    x = x.contiguous()
    N, C, H, W = x.shape
    OH, OW = output_size
    out = torch.empty(N, C, OH, OW, dtype=torch.float32, device=x.device)
    lib = _lib()
    lib.rb_adaptive_avg_pool2d.argtypes = [c_vp, c_vp, c_vp, c_ll, c_int, c_int, c_int, c_int, c_vp]
    check_rc(lib.rb_adaptive_avg_pool2d(ptr(x), None, ptr(out), N * C, H, W, OH, OW, stream_handle(x.device)), "rb_adaptive_avg_pool2d")
    return out


def adaptive_avg_pool2d_backward(dy: torch.Tensor, input_size: tuple[int, int]) -> torch.Tensor:
    """Gradient w.r.t. the ``[N, C, H, W]`` input given ``dy [N, C, OH, OW]`` (gather form, no atomics)."""
    H, W = input_size
    if not dy.is_cuda:
        x = torch.zeros(dy.shape[0], dy.shape[1], H, W, dtype=torch.float32, requires_grad=True)
        torch.nn.functional.adaptive_avg_pool2d(x, dy.shape[-2:]).backward(dy.float())
        return x.grad
    assert dy.dtype == torch.float32 and dy.dim() == 4
    dy = dy.contiguous()
    N, C, OH, OW = dy.shape
    out = torch.empty(N, C, H, W, dtype=torch.float32, device=dy.device)
    lib = _lib()
    lib.rb_adaptive_avg_pool2d.argtypes = [c_vp, c_vp, c_vp, c_ll, c_int, c_int, c_int, c_int, c_vp]
    check_rc(lib.rb_adaptive_avg_pool2d(None, ptr(dy), ptr(out), N * C, H, W, OH, OW, stream_handle(dy.device)),
             "rb_adaptive_avg_pool2d(bwd)")
    return out


def vec_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Element-wise bf16 sum with 16-byte accesses (element count a multiple of 8)."""
    if not a.is_cuda:
        return a + b
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape == b.shape and a.numel() % 8 == 0
    a, b = a.contiguous(), b.contiguous()
    out = torch.empty_like(a)
    lib = _lib()
    lib.rb_vec_add_bf16.argtypes = [c_vp, c_vp, c_vp, c_ll, c_vp]
    check_rc(lib.rb_vec_add_bf16(ptr(a), ptr(b), ptr(out), a.numel(), stream_handle(a.device)), "rb_vec_add_bf16")
    return out
