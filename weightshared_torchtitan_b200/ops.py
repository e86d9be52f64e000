"""Tensor-level wrappers of the C ABI (include/wsl.h).

PyTorch is plumbing here: it owns device memory and the current stream; every function
below extracts raw pointers, pitches and the stream handle and calls straight into
libwsl.so. All launches go on ``torch.cuda.current_stream()``; nothing synchronises.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import WSL_BF16, WSL_F32


# Optional per-launch device timing (bench.py): when a list is installed every wrapper
# brackets its C-ABI call with CUDA events on the launching stream and appends
# (kind, algorithmic_flops, algorithmic_bytes, start_event, end_event).
_TIMING = None


def set_timing(records) -> None:
    """Install (a list) or remove (None) the per-launch timing sink."""
    global _TIMING
    _TIMING = records


def _tic():
    if _TIMING is None:
        return None
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e


# SM reservation window (TrainStep with an overlapped gradient exchange): while a collective
# is estimated to be in flight the library's persistent kernels leave `_RESERVED` SMs free.
# The window is measured in estimated milliseconds of the kernels enqueued after it opened
# (algorithmic FLOPs at ~1.2 PFLOP/s, bytes at ~5 TB/s), because the host runs ahead of the
# device and cannot see when the collective really ends.
_RESERVED = 0
_RESERVE_MS = 0.0


def reserve_sms(n: int, window_ms: float) -> None:
    """Open (or extend by `window_ms`) a window during which launches leave `n` SMs free;
    n <= 0 closes it at once."""
    global _RESERVED, _RESERVE_MS
    if n <= 0:
        if _RESERVED:
            _lib.set_option(_lib.OPT_RESERVED_SMS, 0)
        _RESERVED, _RESERVE_MS = 0, 0.0
        return
    _RESERVE_MS += float(window_ms)
    if _RESERVED != n:
        _lib.set_option(_lib.OPT_RESERVED_SMS, n)
        _RESERVED = n


def _toc(e0, kind: str, flops: float, nbytes: float) -> None:
    global _RESERVE_MS
    if _RESERVED:
        _RESERVE_MS -= max(flops / 1.2e12, nbytes / 5e9)
        if _RESERVE_MS <= 0.0:
            reserve_sms(0, 0.0)
    if e0 is None:
        return
    e1 = torch.cuda.Event(enable_timing=True)
    e1.record()
    _TIMING.append((kind, flops, nbytes, e0, e1))


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return WSL_BF16
    if t.dtype == torch.float32:
        return WSL_F32
    raise TypeError(f"wsl kernels take bfloat16 or float32 tensors, got {t.dtype}")


def _mat(t: torch.Tensor, name: str) -> torch.Tensor:
    """A 2-D CUDA matrix whose last dimension is contiguous (row pitch may exceed width)."""
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the wsl path has no CPU implementation")
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
    if t.shape[1] > 1 and t.stride(1) != 1:
        t = t.contiguous()
    elif t.shape[0] > 1 and t.stride(0) < t.shape[1]:
        t = t.contiguous()
    return t


def _ld(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _same(code: int, *ts: torch.Tensor) -> None:
    for t in ts:
        if _dtype_code(t) != code:
            raise TypeError("all matrices of one wsl call must share a dtype")


def linear_fwd(x: torch.Tensor, W: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """y = x @ W.T (wsl_linear_fwd)."""
    x, W = _mat(x, "x"), _mat(W, "W").contiguous()
    code = _dtype_code(x)
    _same(code, W)
    M, K = x.shape
    N = W.shape[0]
    if W.shape[1] != K:
        raise ValueError("W must be [N, K]")
    y = torch.empty((M, N), device=x.device,
                    dtype=torch.float32 if (out_f32 or code == WSL_F32) else torch.bfloat16)
    _e = _tic()
    st = _lib.lib().wsl_linear_fwd(x.data_ptr(), _ld(x), W.data_ptr(), y.data_ptr(), N, M, N, K,
                                   int(bool(out_f32)), code, _stream())
    _toc(_e, "linear_fwd", 2.0 * M * N * K, x.element_size() * (M * K + N * K) + y.element_size() * M * N)
    _lib.check(st, "wsl_linear_fwd")
    return y


def lora_prepass(x: torch.Tensor, A_cat: torch.Tensor, s: float) -> torch.Tensor:
    """T = s * x @ A_cat.T (wsl_lora_prepass)."""
    x, A_cat = _mat(x, "x"), _mat(A_cat, "A_cat").contiguous()
    code = _dtype_code(x)
    _same(code, A_cat)
    M, K = x.shape
    r_tot = A_cat.shape[0]
    if A_cat.shape[1] != K:
        raise ValueError("A_cat must be [r_tot, K]")
    T = torch.empty((M, r_tot), device=x.device, dtype=x.dtype)
    _e = _tic()
    st = _lib.lib().wsl_lora_prepass(x.data_ptr(), _ld(x), A_cat.data_ptr(), T.data_ptr(), r_tot,
                                     M, K, r_tot, float(s), code, _stream())
    _toc(_e, "prepass_T", 2.0 * M * K * r_tot, x.element_size() * (M * K + r_tot * K + M * r_tot))
    _lib.check(st, "wsl_lora_prepass")
    return T


def lora_linear_fwd(x: torch.Tensor, W: torch.Tensor, T: Optional[torch.Tensor],
                    B: Optional[torch.Tensor]) -> torch.Tensor:
    """y = x @ W.T + T @ B.T with T the scaled pre-pass output (wsl_lora_linear_fwd)."""
    x, W = _mat(x, "x"), _mat(W, "W").contiguous()
    code = _dtype_code(x)
    _same(code, W)
    M, K = x.shape
    N = W.shape[0]
    r = 0
    tp = bp = None
    ldt = 0
    if T is not None:
        T, B = _mat(T, "T"), _mat(B, "B").contiguous()
        _same(code, T, B)
        r = B.shape[1]
        if T.shape != (M, r) or B.shape[0] != N:
            raise ValueError("T must be [M, r] and B [N, r]")
        tp, bp, ldt = T.data_ptr(), B.data_ptr(), _ld(T)
    y = torch.empty((M, N), device=x.device, dtype=x.dtype)
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_fwd(x.data_ptr(), _ld(x), W.data_ptr(), tp, ldt, bp,
                                        y.data_ptr(), N, M, N, K, r, code, _stream())
    _toc(_e, "fwd", 2.0 * M * N * (K + r), x.element_size() * (M * K + N * K + M * r + N * r + M * N))
    _lib.check(st, "wsl_lora_linear_fwd")
    return y


def lora_linear_fwd_group(x: torch.Tensor, Ws, Ts, Bs):
    """y_p = x @ W_p.T + T_p @ B_p.T for projections sharing x and rank, in one launch (bf16)."""
    x = _mat(x, "x")
    code = _dtype_code(x)
    if code != WSL_BF16:
        raise TypeError("the grouped forward launch is the bf16 path")
    n = len(Ws)
    M, K = x.shape
    Ws = [_mat(w, "W").contiguous() for w in Ws]
    Bs = [_mat(b, "B").contiguous() for b in Bs]
    Ts = [_mat(t, "T") for t in Ts]
    vp, ll = ctypes.c_void_p * n, ctypes.c_longlong * n
    w_p, t_p, b_p, y_p = vp(), vp(), vp(), vp()
    ldt, ldy, Ns, rs = ll(), ll(), ll(), ll()
    ys = []
    flops = 0.0
    nbytes = 2.0 * M * K
    for p in range(n):
        _same(code, Ws[p], Bs[p], Ts[p])
        N, r = Ws[p].shape[0], Bs[p].shape[1]
        if Ws[p].shape[1] != K or Ts[p].shape != (M, r) or Bs[p].shape[0] != N:
            raise ValueError("W_p must be [N_p, K], T_p [M, r], B_p [N_p, r]")
        y = torch.empty((M, N), device=x.device, dtype=x.dtype)
        ys.append(y)
        w_p[p], t_p[p], b_p[p], y_p[p] = Ws[p].data_ptr(), Ts[p].data_ptr(), Bs[p].data_ptr(), y.data_ptr()
        ldt[p], ldy[p], Ns[p], rs[p] = _ld(Ts[p]), N, N, r
        flops += 2.0 * M * N * (K + r)
        nbytes += 2.0 * (N * K + M * r + N * r + M * N)
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_fwd_group(n, x.data_ptr(), _ld(x), w_p, t_p, ldt, b_p, y_p, ldy, Ns, rs,
                                              M, K, _stream())
    _toc(_e, "fwd", flops, nbytes)
    _lib.check(st, "wsl_lora_linear_fwd_group")
    return ys


def lora_swiglu_supported(M: int, N: int, K: int, r: int) -> bool:
    """Whether lora_swiglu_fwd covers this shape (wsl_lora_swiglu_supported)."""
    return bool(_lib.lib().wsl_lora_swiglu_supported(M, N, K, r))


def lora_swiglu_fwd(x: torch.Tensor, Wg: torch.Tensor, Wu: torch.Tensor, T_cat: Optional[torch.Tensor],
                    Bg: Optional[torch.Tensor], Bu: Optional[torch.Tensor]):
    """(g, u, h) with g = x Wg^T + T_cat[:, :r] Bg^T, u = x Wu^T + T_cat[:, r:] Bu^T and
    h = silu(g) * u, in one launch (wsl_lora_swiglu_fwd, bf16)."""
    x, Wg, Wu = _mat(x, "x"), _mat(Wg, "W_gate").contiguous(), _mat(Wu, "W_up").contiguous()
    _same(WSL_BF16, x, Wg, Wu)
    M, K = x.shape
    N = Wg.shape[0]
    if Wg.shape != (N, K) or Wu.shape != (N, K):
        raise ValueError("W_gate and W_up must both be [N, K]")
    r = 0
    tp = bgp = bup = None
    ldt = 0
    if T_cat is not None:
        T_cat, Bg, Bu = _mat(T_cat, "T_cat"), _mat(Bg, "B_gate").contiguous(), _mat(Bu, "B_up").contiguous()
        _same(WSL_BF16, T_cat, Bg, Bu)
        r = Bg.shape[1]
        if T_cat.shape != (M, 2 * r) or Bg.shape != (N, r) or Bu.shape != (N, r):
            raise ValueError("T_cat must be [M, 2r], B_gate and B_up [N, r]")
        tp, bgp, bup, ldt = T_cat.data_ptr(), Bg.data_ptr(), Bu.data_ptr(), _ld(T_cat)
    g = torch.empty((M, N), device=x.device, dtype=x.dtype)
    u = torch.empty_like(g)
    h = torch.empty_like(g)
    _e = _tic()
    st = _lib.lib().wsl_lora_swiglu_fwd(x.data_ptr(), _ld(x), Wg.data_ptr(), Wu.data_ptr(), tp, ldt, bgp, bup,
                                        g.data_ptr(), u.data_ptr(), h.data_ptr(), N, M, N, K, r, _stream())
    _toc(_e, "fwd", 4.0 * M * N * (K + r), 2.0 * (M * K + 2 * N * K + 2 * M * r + 2 * N * r + 3 * M * N))
    _lib.check(st, "wsl_lora_swiglu_fwd")
    return g, u, h


def lora_bwd_prepass(dY: torch.Tensor, B: torch.Tensor, s: float,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """U = s * dY @ B (wsl_lora_bwd_prepass). `out` may be a column slice [M, r] of a wider
    buffer (the U of several projections side by side)."""
    dY, B = _mat(dY, "dY"), _mat(B, "B").contiguous()
    code = _dtype_code(dY)
    _same(code, B)
    M, N = dY.shape
    r = B.shape[1]
    if B.shape[0] != N:
        raise ValueError("B must be [N, r]")
    if out is None:
        U = torch.empty((M, r), device=dY.device, dtype=dY.dtype)
    else:
        U = out
        if tuple(U.shape) != (M, r) or U.dtype != dY.dtype or U.stride(1) != 1:
            raise ValueError("out must be an [M, r] view with contiguous rows")
    _e = _tic()
    st = _lib.lib().wsl_lora_bwd_prepass(dY.data_ptr(), _ld(dY), B.data_ptr(), U.data_ptr(), _ld(U),
                                         M, N, r, float(s), code, _stream())
    _toc(_e, "prepass_U", 2.0 * M * N * r, dY.element_size() * (M * N + N * r + M * r))
    _lib.check(st, "wsl_lora_bwd_prepass")
    return U


def lora_linear_bwd_dx(dYs: Sequence[torch.Tensor], Us: Sequence[Optional[torch.Tensor]],
                       Ws: Sequence[torch.Tensor], As: Sequence[Optional[torch.Tensor]]) -> torch.Tensor:
    """dX = sum_p dY_p @ W_p + U_p @ A_p for projections that read the same x."""
    n = len(dYs)
    dYs = [_mat(t, "dY") for t in dYs]
    Ws = [_mat(t, "W").contiguous() for t in Ws]
    code = _dtype_code(dYs[0])
    M = dYs[0].shape[0]
    K = Ws[0].shape[1]
    keep = []
    vp = ctypes.c_void_p * n
    ll = ctypes.c_longlong * n
    dy_p, u_p, w_p, a_p = vp(), vp(), vp(), vp()
    lddy, ldu, Ns, rs = ll(), ll(), ll(), ll()
    for p in range(n):
        _same(code, dYs[p], Ws[p])
        if dYs[p].shape[0] != M or Ws[p].shape != (dYs[p].shape[1], K):
            raise ValueError("dY_p must be [M, N_p] and W_p [N_p, K]")
        dy_p[p], lddy[p] = dYs[p].data_ptr(), _ld(dYs[p])
        w_p[p], Ns[p] = Ws[p].data_ptr(), Ws[p].shape[0]
        if Us[p] is not None:
            U, A = _mat(Us[p], "U"), _mat(As[p], "A").contiguous()
            _same(code, U, A)
            if U.shape != (M, A.shape[0]) or A.shape[1] != K:
                raise ValueError("U_p must be [M, r_p] and A_p [r_p, K]")
            keep += [U, A]
            u_p[p], ldu[p], a_p[p], rs[p] = U.data_ptr(), _ld(U), A.data_ptr(), A.shape[0]
        else:
            u_p[p], ldu[p], a_p[p], rs[p] = None, 0, None, 0
    dX = torch.empty((M, K), device=dYs[0].device, dtype=dYs[0].dtype)
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_bwd_dx(n, dy_p, lddy, u_p, ldu, w_p, a_p, Ns, rs, dX.data_ptr(),
                                           K, M, K, code, _stream())
    _toc(_e, "dx", 2.0 * M * K * sum(int(Ns[p]) + int(rs[p]) for p in range(n)), dX.element_size() * (M * K + sum((M + K) * (int(Ns[p]) + int(rs[p])) for p in range(n))))
    _lib.check(st, "wsl_lora_linear_bwd_dx")
    return dX


def swiglu_bwd_in_dx_supported(M: int, N: int, K: int, r: int) -> bool:
    """Whether lora_linear_bwd_dx_swiglu covers this shape (K = the MLP's inner width)."""
    return bool(_lib.lib().wsl_swiglu_bwd_in_dx_supported(M, N, K, r))


def lora_linear_bwd_dx_swiglu(dY: torch.Tensor, U: Optional[torch.Tensor], W: torch.Tensor,
                              A: Optional[torch.Tensor], g: torch.Tensor, u: torch.Tensor):
    """(d gate, d up) from dh = dY @ W + U @ A without writing dh: the down projection's input
    gradient with the SwiGLU backward in its epilogue (wsl_lora_linear_bwd_dx_swiglu, bf16)."""
    dY, W = _mat(dY, "dY"), _mat(W, "W").contiguous()
    g, u = _mat(g, "g").contiguous(), _mat(u, "u").contiguous()
    _same(WSL_BF16, dY, W, g, u)
    M, N = dY.shape
    K = W.shape[1]
    if W.shape[0] != N or g.shape != (M, K) or u.shape != (M, K):
        raise ValueError("W must be [N, K], g and u [M, K]")
    r = 0
    up = ap = None
    ldu = 0
    if U is not None:
        U, A = _mat(U, "U"), _mat(A, "A").contiguous()
        _same(WSL_BF16, U, A)
        r = A.shape[0]
        if U.shape != (M, r) or A.shape[1] != K:
            raise ValueError("U must be [M, r] and A [r, K]")
        up, ap, ldu = U.data_ptr(), A.data_ptr(), _ld(U)
    dg, du = torch.empty_like(g), torch.empty_like(u)
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_bwd_dx_swiglu(dY.data_ptr(), _ld(dY), up, ldu, W.data_ptr(), ap, g.data_ptr(),
                                                  u.data_ptr(), dg.data_ptr(), du.data_ptr(), K, M, N, K, r,
                                                  _stream())
    _toc(_e, "dx", 2.0 * M * K * (N + r), 2.0 * (M * N + N * K + M * r + r * K + 4 * M * K))
    _lib.check(st, "wsl_lora_linear_bwd_dx_swiglu")
    return dg, du


def lora_linear_bwd_dw(dY: torch.Tensor, U: Optional[torch.Tensor], x: torch.Tensor,
                       T: Optional[torch.Tensor], dW: Optional[torch.Tensor],
                       dA: Optional[torch.Tensor], dB: Optional[torch.Tensor]) -> None:
    """dW += dY.T @ x, dA += U.T @ x, dB += dY.T @ T, in place into fp32 buffers."""
    dY, x = _mat(dY, "dY"), _mat(x, "x")
    code = _dtype_code(dY)
    _same(code, x)
    M, N = dY.shape
    K = x.shape[1]
    if x.shape[0] != M:
        raise ValueError("x must be [M, K]")
    r = 0
    up = tp = None
    ldu = ldt = 0
    if U is not None:
        U = _mat(U, "U")
        _same(code, U)
        r, up, ldu = U.shape[1], U.data_ptr(), _ld(U)
    if T is not None:
        T = _mat(T, "T")
        _same(code, T)
        r, tp, ldt = T.shape[1], T.data_ptr(), _ld(T)
    for g, shape, nm in ((dW, (N, K), "dW"), (dA, (r, K), "dA"), (dB, (N, r), "dB")):
        if g is not None:
            if g.dtype != torch.float32 or not g.is_contiguous() or tuple(g.shape) != shape:
                raise ValueError(f"{nm} must be a contiguous float32 tensor of shape {shape}")
    ws_bytes = 0
    ws = None
    if code == WSL_BF16:
        ws_bytes = int(_lib.lib().wsl_bwd_dw_workspace_bytes(M, N, K, r, int(dW is not None),
                                                             int(dA is not None), int(dB is not None)))
        if ws_bytes:
            ws = torch.empty(ws_bytes // 4, device=dY.device, dtype=torch.float32)
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_bwd_dw(
        dY.data_ptr(), _ld(dY), up, ldu, x.data_ptr(), _ld(x), tp, ldt,
        dW.data_ptr() if dW is not None else None,
        dA.data_ptr() if dA is not None else None,
        dB.data_ptr() if dB is not None else None,
        M, N, K, r, ws.data_ptr() if ws is not None else None, ws_bytes, code, _stream())
    _toc(_e, "dw", 2.0 * M * ((N * K if dW is not None else 0) + (r * K if dA is not None else 0) + (N * r if dB is not None else 0)), dY.element_size() * (M * N + M * K + 2 * M * r) + 8.0 * ((N * K if dW is not None else 0) + (r * K if dA is not None else 0) + (N * r if dB is not None else 0)))
    _lib.check(st, "wsl_lora_linear_bwd_dw")


def lora_linear_bwd_dw_group(dYs, Us, x, Ts, dWs, dAs, dBs) -> None:
    """One launch for the weight gradients of projections that read the same x (bf16):
    dW_p += dY_p.T @ x, dA_p += U_p.T @ x, dB_p += dY_p.T @ T_p, all fp32 in place."""
    n = len(dYs)
    dYs = [_mat(t, "dY") for t in dYs]
    x = _mat(x, "x")
    code = _dtype_code(x)
    if code != WSL_BF16:
        raise TypeError("the grouped weight-gradient launch is the bf16 path")
    M, K = x.shape
    vp, ll = ctypes.c_void_p * n, ctypes.c_longlong * n
    dy_p, u_p, t_p, dw_p, da_p, db_p = vp(), vp(), vp(), vp(), vp(), vp()
    lddy, ldu, ldt, Ns, rs = ll(), ll(), ll(), ll(), ll()
    keep = []
    flops = 0.0
    nbytes = 2.0 * M * K
    for p in range(n):
        _same(code, dYs[p])
        N = dYs[p].shape[1]
        r = 0
        dy_p[p], lddy[p], Ns[p] = dYs[p].data_ptr(), _ld(dYs[p]), N
        if Us[p] is not None:
            U, T = _mat(Us[p], "U"), _mat(Ts[p], "T")
            keep += [U, T]
            r = U.shape[1]
            u_p[p], ldu[p], t_p[p], ldt[p] = U.data_ptr(), _ld(U), T.data_ptr(), _ld(T)
        else:
            u_p[p], ldu[p], t_p[p], ldt[p] = None, 0, None, 0
        rs[p] = r
        for gbuf, shape, nm in ((dWs[p], (N, K), "dW"), (dAs[p], (r, K), "dA"), (dBs[p], (N, r), "dB")):
            if gbuf is not None and (gbuf.dtype != torch.float32 or not gbuf.is_contiguous()
                                     or tuple(gbuf.shape) != shape):
                raise ValueError(f"{nm} must be a contiguous float32 tensor of shape {shape}")
        dw_p[p] = dWs[p].data_ptr()
        da_p[p] = dAs[p].data_ptr() if dAs[p] is not None else None
        db_p[p] = dBs[p].data_ptr() if dBs[p] is not None else None
        flops += 2.0 * M * (N * K + r * K + N * r)
        nbytes += 2.0 * (M * N + 2 * M * r) + 8.0 * (N * K + r * K + N * r)
    ws_bytes = int(_lib.lib().wsl_bwd_dw_group_workspace_bytes(n, Ns, rs, M, K))
    ws = torch.empty(ws_bytes // 4, device=x.device, dtype=torch.float32) if ws_bytes else None
    _e = _tic()
    st = _lib.lib().wsl_lora_linear_bwd_dw_group(
        n, dy_p, lddy, u_p, ldu, x.data_ptr(), _ld(x), t_p, ldt, dw_p, da_p, db_p, Ns, rs, M, K,
        ws.data_ptr() if ws is not None else None, ws_bytes, _stream())
    _toc(_e, "dw", flops, nbytes)
    _lib.check(st, "wsl_lora_linear_bwd_dw_group")


MERGE_RANKS = (8, 16, 32, 64, 128)   # ranks wsl_lora_merge_weight is built for


def lora_merge_weight(Ws, As, Bs, s: float) -> list:
    """W_eff_p = bf16(W_p + s B_p A_p) for projections with the same input width and rank, one
    launch."""
    n = len(Ws)
    Ws = [_mat(t, "W").contiguous() for t in Ws]
    As = [_mat(t, "A").contiguous() for t in As]
    Bs = [_mat(t, "B").contiguous() for t in Bs]
    K = Ws[0].shape[1]
    vp, ll = ctypes.c_void_p * n, ctypes.c_longlong * n
    w_p, a_p, b_p, o_p, Ns = vp(), vp(), vp(), vp(), ll()
    r0 = As[0].shape[0]
    outs = []
    flops = nbytes = 0.0
    for p in range(n):
        if _dtype_code(Ws[p]) != WSL_BF16:
            raise TypeError("lora_merge_weight is a bf16 operation")
        _same(WSL_BF16, As[p], Bs[p])
        N = Ws[p].shape[0]
        r = As[p].shape[0]
        if Ws[p].shape != (N, K) or As[p].shape != (r, K) or Bs[p].shape != (N, r):
            raise ValueError(f"shapes W{tuple(Ws[p].shape)} A{tuple(As[p].shape)} B{tuple(Bs[p].shape)} "
                             "do not fit W + s B A")
        out = torch.empty_like(Ws[p])
        outs.append(out)
        if r != r0:
            raise ValueError("projections merged in one launch must share the rank")
        w_p[p], a_p[p], b_p[p], o_p[p], Ns[p] = (Ws[p].data_ptr(), As[p].data_ptr(), Bs[p].data_ptr(),
                                                out.data_ptr(), N)
        flops += 2.0 * N * K * r
        nbytes += 4.0 * N * K
    _e = _tic()
    st = _lib.lib().wsl_lora_merge_weight(n, w_p, a_p, b_p, o_p, Ns, K, r0, float(s), _stream())
    _toc(_e, "merge_weight", flops, nbytes)
    _lib.check(st, "wsl_lora_merge_weight")
    return outs


def bwd_dw_layer_group(dYs, x, dWs) -> list:
    """dW_p += dY_p.T @ x (fp32, in place) for projections that read the same x, one launch;
    returns the bf16 matrices dWl_p = dY_p.T @ x of this call alone."""
    n = len(dYs)
    dYs = [_mat(t, "dY") for t in dYs]
    x = _mat(x, "x")
    if _dtype_code(x) != WSL_BF16:
        raise TypeError("bwd_dw_layer_group is the bf16 path")
    M, K = x.shape
    vp, ll = ctypes.c_void_p * n, ctypes.c_longlong * n
    dy_p, dw_p, dwl_p, lddy, Ns, rs = vp(), vp(), vp(), ll(), ll(), ll()
    dWls = []
    flops = 0.0
    nbytes = 2.0 * M * K
    for p in range(n):
        _same(WSL_BF16, dYs[p])
        N = dYs[p].shape[1]
        g = dWs[p]
        if g.dtype != torch.float32 or not g.is_contiguous() or tuple(g.shape) != (N, K):
            raise ValueError(f"dW must be a contiguous float32 tensor of shape {(N, K)}")
        dWl = torch.empty((N, K), device=x.device, dtype=torch.bfloat16)
        dWls.append(dWl)
        dy_p[p], lddy[p], Ns[p], rs[p] = dYs[p].data_ptr(), _ld(dYs[p]), N, 0
        dw_p[p], dwl_p[p] = g.data_ptr(), dWl.data_ptr()
        flops += 2.0 * M * N * K
        nbytes += 2.0 * M * N + 10.0 * N * K
    ws_bytes = int(_lib.lib().wsl_bwd_dw_group_workspace_bytes(n, Ns, rs, M, K))
    ws = torch.empty(ws_bytes // 4, device=x.device, dtype=torch.float32) if ws_bytes else None
    _e = _tic()
    st = _lib.lib().wsl_bwd_dw_layer_group(n, dy_p, lddy, x.data_ptr(), _ld(x), dw_p, dwl_p, Ns, M, K,
                                           ws.data_ptr() if ws is not None else None, ws_bytes, _stream())
    _toc(_e, "dw", flops, nbytes)
    _lib.check(st, "wsl_bwd_dw_layer_group")
    return dWls


MAX_ADAPTER_PROJ = 9   # WSL_MAX_ADAPTER_PROJ


def lora_adapter_grads_from_dw(dWls, As, Bs, dAs, dBs, s: float) -> None:
    """dA_p += s B_p.T @ dWl_p, dB_p += s dWl_p @ A_p.T (fp32, in place) for up to
    MAX_ADAPTER_PROJ projections of any sizes in two launches."""
    n = len(dWls)
    vp, ll = ctypes.c_void_p * n, ctypes.c_longlong * n
    g_p, a_p, b_p, da_p, db_p, Ns, Ks, rs = vp(), vp(), vp(), vp(), vp(), ll(), ll(), ll()
    keep = []
    flops = 0.0
    nbytes = 0.0
    for p in range(n):
        G, A, B = _mat(dWls[p], "dWl"), _mat(As[p], "A").contiguous(), _mat(Bs[p], "B").contiguous()
        _same(WSL_BF16, G, A, B)
        if not G.is_contiguous():
            raise ValueError("dWl must be dense")
        N, r = B.shape
        K = G.shape[1]
        if G.shape != (N, K) or A.shape != (r, K):
            raise ValueError("shapes of dWl, A, B do not fit")
        for gbuf, shape, nm in ((dAs[p], (r, K), "dA"), (dBs[p], (N, r), "dB")):
            if gbuf.dtype != torch.float32 or not gbuf.is_contiguous() or tuple(gbuf.shape) != shape:
                raise ValueError(f"{nm} must be a contiguous float32 tensor of shape {shape}")
        keep += [G, A, B]
        g_p[p], a_p[p], b_p[p] = G.data_ptr(), A.data_ptr(), B.data_ptr()
        da_p[p], db_p[p], Ns[p], Ks[p], rs[p] = dAs[p].data_ptr(), dBs[p].data_ptr(), N, K, r
        flops += 4.0 * N * K * r
        nbytes += 4.0 * N * K
    ws_bytes = int(_lib.lib().wsl_adapter_grads_workspace_bytes(n, Ns, Ks, rs))
    ws = torch.empty(ws_bytes // 4, device=dWls[0].device, dtype=torch.float32) if ws_bytes else None
    _e = _tic()
    st = _lib.lib().wsl_lora_adapter_grads_from_dw(n, g_p, a_p, b_p, da_p, db_p, Ns, Ks, rs, float(s),
                                                   ws.data_ptr() if ws is not None else None, ws_bytes,
                                                   _stream())
    _toc(_e, "adapter_grads", flops, nbytes)
    _lib.check(st, "wsl_lora_adapter_grads_from_dw")


def embed_gather(tokens: torch.Tensor, E_small: torch.Tensor) -> torch.Tensor:
    """G[m] = E_small[tokens[m]] (bit-exact row copy)."""
    tok = tokens.reshape(-1)
    if tok.dtype != torch.int64 or not tok.is_cuda:
        raise TypeError("tokens must be a CUDA int64 tensor")
    tok = tok.contiguous()
    E = _mat(E_small, "E_small").contiguous()
    V, r_e = E.shape
    G = torch.empty((tok.numel(), r_e), device=E.device, dtype=E.dtype)
    _e = _tic()
    st = _lib.lib().wsl_embed_gather(tok.data_ptr(), E.data_ptr(), G.data_ptr(), tok.numel(), V, r_e,
                                     _dtype_code(E), _stream())
    _toc(_e, "embed_gather", 0.0, 8.0 * tok.numel() + 2.0 * E.element_size() * tok.numel() * r_e)
    _lib.check(st, "wsl_embed_gather")
    return G


# Output widths up to which the row gather runs inside the GEMM's TMA producer (embed_fwd,
# embed_bwd_dproj). Measured on B200 at 16384 tokens, r_e = 1024, d = 4096 (16 column tiles):
# gather inside the GEMM 288 us forward / 398 us backward, against 16 us for the gather kernel
# plus 105 us for the plain GEMM; the gather4 instructions (4 rows x 128 B each) set the pace
# and repeat per column tile, so the fused form is kept where there are few column tiles.
EMBED_GATHER_IN_GEMM_MAX_DIM = 1024


def embed_gather_in_gemm_pays(d: int) -> bool:
    return int(d) <= EMBED_GATHER_IN_GEMM_MAX_DIM


def embed_fwd(tokens: torch.Tensor, E_small: torch.Tensor, P: torch.Tensor) -> torch.Tensor:
    """h = E_small[tokens] @ P.T with the row gather inside the GEMM's TMA producer (bf16)."""
    tok = tokens.reshape(-1)
    if tok.dtype != torch.int64 or not tok.is_cuda:
        raise TypeError("tokens must be a CUDA int64 tensor")
    tok = tok.contiguous()
    E, P = _mat(E_small, "E_small").contiguous(), _mat(P, "P").contiguous()
    if E.dtype != torch.bfloat16 or P.dtype != torch.bfloat16:
        raise TypeError("embed_fwd is the bf16 path; fp32 uses embed_gather + linear_fwd")
    V, r_e = E.shape
    d = P.shape[0]
    M = tok.numel()
    h = torch.empty((M, d), device=E.device, dtype=E.dtype)
    _e = _tic()
    st = _lib.lib().wsl_embed_fwd(tok.data_ptr(), E.data_ptr(), P.data_ptr(), h.data_ptr(), d, M, V, r_e, d,
                                  _stream())
    _toc(_e, "embed_fwd", 2.0 * M * r_e * d, 8.0 * M + 2.0 * (M * r_e + r_e * d + M * d))
    _lib.check(st, "wsl_embed_fwd")
    return h


def embed_bwd_dproj(tokens: torch.Tensor, dH: torch.Tensor, E_small: torch.Tensor, dP: torch.Tensor) -> None:
    """dP += dH.T @ E_small[tokens] (fp32 in place), gathering inside the GEMM."""
    tok = tokens.reshape(-1).contiguous()
    dH = _mat(dH, "dH")
    E = _mat(E_small, "E_small").contiguous()
    V, r_e = E.shape
    M, d = dH.shape
    if dP.dtype != torch.float32 or not dP.is_contiguous() or tuple(dP.shape) != (d, r_e):
        raise ValueError("dP must be contiguous float32 [d, r_e]")
    ws = torch.empty(16 * d * r_e, device=dH.device, dtype=torch.float32)
    _e = _tic()
    st = _lib.lib().wsl_embed_bwd_dproj(tok.data_ptr(), dH.data_ptr(), _ld(dH), E.data_ptr(), dP.data_ptr(),
                                        M, V, r_e, d, ws.data_ptr(), ws.numel() * 4, _stream())
    _toc(_e, "embed_dproj", 2.0 * M * r_e * d, 8.0 * M + 2.0 * (M * r_e + M * d) + 8.0 * r_e * d)
    _lib.check(st, "wsl_embed_bwd_dproj")


def embed_scatter_add(tokens: torch.Tensor, dG: torch.Tensor, dE: torch.Tensor) -> None:
    """dE[tokens[m]] += dG[m] into a contiguous fp32 [V, r_e] buffer."""
    tok = tokens.reshape(-1).contiguous()
    dG = _mat(dG, "dG").contiguous()
    if dE.dtype != torch.float32 or not dE.is_contiguous():
        raise ValueError("dE must be contiguous float32")
    V, r_e = dE.shape
    _e = _tic()
    st = _lib.lib().wsl_embed_scatter_add(tok.data_ptr(), dG.data_ptr(), dE.data_ptr(), tok.numel(),
                                          V, r_e, _dtype_code(dG), _stream())
    _toc(_e, "embed_scatter", 0.0, 8.0 * tok.numel() + (dG.element_size() + 8.0) * tok.numel() * r_e)
    _lib.check(st, "wsl_embed_scatter_add")


# ------------------------------------------------ rows either side of the projections
def ce_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, scale: float,
               scale_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place: logits <- scale * scale_dev * (softmax - onehot); returns per-row loss (fp32).
    `scale_dev` is an optional one-element CUDA float32 tensor (a factor that exists only on
    the device, such as 1 / the number of counted rows)."""
    logits = _mat(logits, "logits")
    lab = labels.reshape(-1)
    if lab.dtype != torch.int64 or not lab.is_cuda or lab.numel() != logits.shape[0]:
        raise TypeError("labels must be a CUDA int64 tensor with one entry per row")
    lab = lab.contiguous()
    rows, V = logits.shape
    row_loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    if scale_dev is not None and (scale_dev.dtype != torch.float32 or not scale_dev.is_cuda
                                  or scale_dev.numel() != 1):
        raise TypeError("scale_dev must be a one-element CUDA float32 tensor")
    _e = _tic()
    st = _lib.lib().wsl_ce_fwd_bwd(logits.data_ptr(), _ld(logits), lab.data_ptr(), row_loss.data_ptr(),
                                   rows, V, float(scale), scale_dev.data_ptr() if scale_dev is not None else None,
                                   _dtype_code(logits), _stream())
    _toc(_e, "ce", 0.0, 3.0 * logits.element_size() * rows * V)
    _lib.check(st, "wsl_ce_fwd_bwd")
    return row_loss


def swiglu_fwd(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(gate)
    _e = _tic()
    st = _lib.lib().wsl_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(),
                                   _dtype_code(gate), _stream())
    _toc(_e, "swiglu_fwd", 0.0, 3.0 * gate.element_size() * gate.numel())
    _lib.check(st, "wsl_swiglu_fwd")
    return out


def swiglu_bwd(dout: torch.Tensor, gate: torch.Tensor, up: torch.Tensor):
    dout = dout.contiguous()
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    _e = _tic()
    st = _lib.lib().wsl_swiglu_bwd(dout.data_ptr(), gate.data_ptr(), up.data_ptr(), dg.data_ptr(),
                                   du.data_ptr(), gate.numel(), _dtype_code(gate), _stream())
    _toc(_e, "swiglu_bwd", 0.0, 5.0 * gate.element_size() * gate.numel())
    _lib.check(st, "wsl_swiglu_bwd")
    return dg, du


def rmsnorm_supported(D: int, dtype: torch.dtype, rope: bool = False) -> bool:
    """Row widths the fused RMSNorm kernels cover (see wsl_rmsnorm_fwd in include/wsl.h)."""
    nv = 8 if dtype == torch.bfloat16 else 4
    if D % nv:
        return False
    lanes = D // nv
    if rope:
        return 2 <= lanes <= 32 and lanes & (lanes - 1) == 0
    if lanes >= 32:
        # 10 and 16 vectors per lane (hidden sizes 2560, 4096): bf16, dense rows only
        return D % (32 * nv) == 0 and D // (32 * nv) in ((1, 2, 4, 8, 10, 16) if nv == 8 else (1, 2, 4, 8))
    return lanes & (lanes - 1) == 0


def rmsnorm_fwd(x2: torch.Tensor, w: torch.Tensor, eps: float, rope=None):
    """x2 [rows, D]; w fp32 [D]; rope = (cos, sin, heads, seq) with fp32 [seq, D] tables.
    Returns (y, rstd)."""
    x2 = _mat(x2, "x")
    rows, D = x2.shape
    if D > 2048:
        x2 = x2.contiguous()   # rows this wide are covered by the dense-row kernels only
    y = torch.empty((rows, D), device=x2.device, dtype=x2.dtype)
    rstd = torch.empty(rows, device=x2.device, dtype=torch.float32)
    cs = sn = None
    heads = seq = 0
    if rope is not None:
        cos, sin, heads, seq = rope
        cs, sn = cos.data_ptr(), sin.data_ptr()
    _e = _tic()
    st = _lib.lib().wsl_rmsnorm_fwd(x2.data_ptr(), _ld(x2), w.data_ptr(), y.data_ptr(), D, rstd.data_ptr(),
                                    rows, D, float(eps), cs, sn, heads, seq, _dtype_code(x2), _stream())
    _toc(_e, "rmsnorm_fwd", 0.0, 2.0 * x2.element_size() * rows * D)
    _lib.check(st, "wsl_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dw: Optional[torch.Tensor], rope=None) -> torch.Tensor:
    dy2, x2 = _mat(dy2, "dy"), _mat(x2, "x")
    rows, D = x2.shape
    if D > 2048:
        dy2, x2 = dy2.contiguous(), x2.contiguous()
    dx = torch.empty((rows, D), device=x2.device, dtype=x2.dtype)
    cs = sn = None
    heads = seq = 0
    if rope is not None:
        cos, sin, heads, seq = rope
        cs, sn = cos.data_ptr(), sin.data_ptr()
    _e = _tic()
    st = _lib.lib().wsl_rmsnorm_bwd(dy2.data_ptr(), _ld(dy2), x2.data_ptr(), _ld(x2), w.data_ptr(),
                                    rstd.data_ptr(), dx.data_ptr(), D,
                                    dw.data_ptr() if dw is not None else None, rows, D, cs, sn, heads, seq,
                                    _dtype_code(x2), _stream())
    _toc(_e, "rmsnorm_bwd", 0.0, 3.0 * x2.element_size() * rows * D)
    _lib.check(st, "wsl_rmsnorm_bwd")
    return dx


def add_rmsnorm_fwd(x2: torch.Tensor, res2: torch.Tensor, w: torch.Tensor, eps: float):
    """h = x + res, y = RMSNorm(h) * w in one pass (dense rows). Returns (h, y, rstd)."""
    x2, res2 = _mat(x2, "x").contiguous(), _mat(res2, "res").contiguous()
    _same(_dtype_code(x2), res2)
    rows, D = x2.shape
    if res2.shape != x2.shape:
        raise ValueError("x and res must have the same shape")
    h = torch.empty_like(x2)
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, device=x2.device, dtype=torch.float32)
    _e = _tic()
    st = _lib.lib().wsl_add_rmsnorm_fwd(x2.data_ptr(), res2.data_ptr(), w.data_ptr(), h.data_ptr(), y.data_ptr(),
                                        rstd.data_ptr(), rows, D, float(eps), _dtype_code(x2), _stream())
    _toc(_e, "rmsnorm_fwd", 0.0, 4.0 * x2.element_size() * rows * D)
    _lib.check(st, "wsl_add_rmsnorm_fwd")
    return h, y, rstd


def add_rmsnorm_bwd(dy2: torch.Tensor, h2: torch.Tensor, dres2: torch.Tensor, w: torch.Tensor,
                    rstd: torch.Tensor, dw: Optional[torch.Tensor]) -> torch.Tensor:
    """dx = dRMSNorm(dy; h, w, rstd) + dres (dense rows); dw accumulates in place."""
    dy2, h2, dres2 = _mat(dy2, "dy").contiguous(), _mat(h2, "h").contiguous(), _mat(dres2, "dres").contiguous()
    _same(_dtype_code(h2), dy2, dres2)
    rows, D = h2.shape
    dx = torch.empty_like(h2)
    _e = _tic()
    st = _lib.lib().wsl_add_rmsnorm_bwd(dy2.data_ptr(), h2.data_ptr(), dres2.data_ptr(), w.data_ptr(),
                                        rstd.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr() if dw is not None else None, rows, D,
                                        _dtype_code(h2), _stream())
    _toc(_e, "rmsnorm_bwd", 0.0, 4.0 * h2.element_size() * rows * D)
    _lib.check(st, "wsl_add_rmsnorm_bwd")
    return dx


SUMSQ_PARTIALS = 1184   # WSL_SUMSQ_PARTIALS


def grad_sumsq_partials(g: torch.Tensor, partials: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Partial sums of g^2 over a flat fp32 buffer (fixed grid, fixed order); their sum is the
    squared global gradient norm."""
    if not g.is_cuda or g.dtype != torch.float32 or not g.is_contiguous():
        raise TypeError("g must be a contiguous CUDA float32 tensor")
    if partials is None:
        partials = torch.empty(SUMSQ_PARTIALS, device=g.device, dtype=torch.float32)
    _e = _tic()
    st = _lib.lib().wsl_grad_sumsq_partials(g.data_ptr(), g.numel(), partials.data_ptr(), _stream())
    _toc(_e, "grad_sumsq", 0.0, 4.0 * g.numel())
    _lib.check(st, "wsl_grad_sumsq_partials")
    return partials


def adamw_flat_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                    p_copy: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float,
                    weight_decay: float, step: int, partials: Optional[torch.Tensor],
                    max_norm: Optional[float]) -> None:
    """Clip by the global norm (from `partials`), AdamW step number `step` (1-based) on the flat
    fp32 buffers, and the bf16 copy of the new parameters, in one pass."""
    for t in (p, g, m, v):
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != p.numel():
            raise TypeError("p, g, m, v must be contiguous CUDA float32 tensors of one size")
    if p_copy is not None and (p_copy.dtype != torch.bfloat16 or p_copy.numel() != p.numel()
                               or not p_copy.is_contiguous()):
        raise TypeError("p_copy must be a contiguous bfloat16 tensor of the size of p")
    clip = max_norm is not None and max_norm > 0
    _e = _tic()
    st = _lib.lib().wsl_adamw_flat_step(
        p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
        p_copy.data_ptr() if p_copy is not None else None, p.numel(), float(lr), float(beta1), float(beta2),
        float(eps), float(weight_decay), 1.0 - beta1 ** step, 1.0 - beta2 ** step,
        partials.data_ptr() if clip else None, partials.numel() if clip else 0,
        float(max_norm) if clip else 0.0, _stream())
    _toc(_e, "adamw", 0.0, 30.0 * p.numel())
    _lib.check(st, "wsl_adamw_flat_step")
