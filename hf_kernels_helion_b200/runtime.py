"""Host-side launch helpers: argument checks, workspace and status word, ctypes calls.

Everything below enqueues work on torch's current CUDA stream and returns without
synchronising, like the reference op (which launches a Triton kernel on the current
stream: torch-ext/finegrained_fp8_helion/fp8.py:19-39).
"""
from __future__ import annotations

import os

import torch

from . import _lib

FP8 = torch.float8_e4m3fn
_OUT_CODES = {torch.bfloat16: _lib.OUT_BF16, torch.float32: _lib.OUT_FP32}

# (device index, stream handle) -> uint8 workspace tensor; device index -> int32 status word
_workspaces: dict = {}
_status_words: dict = {}


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU implementation")


def _row_major(t: torch.Tensor, align_elems: int) -> torch.Tensor:
    """Return t itself if it is a row-major view the kernels can address (unit inner stride,
    row stride and base address multiples of `align_elems` elements), else a contiguous copy."""
    rows, cols = t.shape
    ok = cols <= 1 or t.stride(1) == 1
    if rows > 1:
        ok = ok and t.stride(0) >= cols and t.stride(0) % align_elems == 0
    ok = ok and t.data_ptr() % (align_elems * t.element_size()) == 0
    return t if ok else t.contiguous()


def _ld(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], 1)


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel reported a bounded-wait timeout since the last check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"b200fp8 kernel reported device status {code} (1 = bounded wait timed out); "
                           "the output of that launch is invalid")


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def resolve_variant(variant) -> int:
    if variant is None:
        variant = os.environ.get("B200FP8_VARIANT", "auto")
    if isinstance(variant, str):
        try:
            return _lib.VARIANT_NAMES[variant.lower()]
        except KeyError:
            raise ValueError(f"unknown variant {variant!r}; expected one of {sorted(_lib.VARIANT_NAMES)}") from None
    return int(variant)


def gemm(A, B, As, Bs, block_n: int, block_k: int, out_dtype: torch.dtype, variant=None, out=None) -> torch.Tensor:
    if int(block_n) != 128 or int(block_k) != 128:
        raise ValueError(f"block_size must be [128, 128], got [{block_n}, {block_k}]")
    if out_dtype not in _OUT_CODES:
        raise ValueError(f"output dtype must be torch.bfloat16 or torch.float32, got {out_dtype}")
    for name, t in (("A", A), ("B", B), ("As", As), ("Bs", Bs)):
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
        if t.device != A.device:
            raise ValueError("all tensors must be on the same device")
    if A.dtype != FP8 or B.dtype != FP8:
        raise ValueError(f"A and B must be torch.float8_e4m3fn, got {A.dtype} and {B.dtype}")
    if As.dtype != torch.float32 or Bs.dtype != torch.float32:
        raise ValueError(f"As and Bs must be torch.float32, got {As.dtype} and {Bs.dtype}")
    M, K = A.shape
    N, Kb = B.shape
    if K != Kb:
        raise ValueError(f"A is [M={M}, K={K}] but B is [N={N}, K={Kb}]")
    kblocks, nblocks = -(-K // 128), -(-N // 128)
    if tuple(As.shape) != (M, kblocks):
        raise ValueError(f"As must be [M, ceil(K/128)] = [{M}, {kblocks}], got {tuple(As.shape)}")
    if tuple(Bs.shape) != (nblocks, kblocks):
        raise ValueError(f"Bs must be [ceil(N/128), ceil(K/128)] = [{nblocks}, {kblocks}], got {tuple(Bs.shape)}")

    _require_cuda(A, "A")
    dev = A.device
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    else:
        if tuple(out.shape) != (M, N) or out.dtype != out_dtype or out.device != dev:
            raise ValueError("out has the wrong shape, dtype or device")
        if N > 1 and out.stride(1) != 1:
            raise ValueError("out must have unit stride along N")
    if M == 0 or N == 0:
        return out

    lib = _lib.load()
    A_, B_ = _row_major(A, 16), _row_major(B, 16)
    As_, Bs_ = _row_major(As, 1), _row_major(Bs, 1)
    v = resolve_variant(variant)
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200fp8_gemm_workspace_bytes(M, N, K, v))
        if ws_bytes < 0:
            _lib.check(-ws_bytes, "b200fp8_gemm_workspace_bytes")
        ws = _workspace(dev, ws_bytes) if ws_bytes > 0 else None
        st = lib.b200fp8_gemm(
            A_.data_ptr(), B_.data_ptr(), As_.data_ptr(), Bs_.data_ptr(), out.data_ptr(),
            M, N, K, _ld(A_), _ld(B_), _ld(As_), _ld(Bs_), _ld(out),
            _OUT_CODES[out_dtype], v,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "b200fp8_gemm")
    return out


def gemm_rowscale(A, B, As, Bs, block_k: int, out_dtype: torch.dtype) -> torch.Tensor:
    """C = A @ B.T with As [M, ceil(K/128)] and one B scale per ROW of B, Bs [N, ceil(K/128)]
    (b200fp8_gemm_rowscale; the operand layout of deep-gemm-helion's gemm_fp8_fp8_bf16_nt)."""
    if int(block_k) != 128:
        raise ValueError(f"block_size must be 128, got {block_k}")
    if out_dtype not in _OUT_CODES:
        raise ValueError(f"output dtype must be torch.bfloat16 or torch.float32, got {out_dtype}")
    for name, t in (("A", A), ("B", B), ("As", As), ("Bs", Bs)):
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
        if t.device != A.device:
            raise ValueError("all tensors must be on the same device")
    if A.dtype != FP8 or B.dtype != FP8:
        raise ValueError(f"A and B must be torch.float8_e4m3fn, got {A.dtype} and {B.dtype}")
    if As.dtype != torch.float32 or Bs.dtype != torch.float32:
        raise ValueError(f"As and Bs must be torch.float32, got {As.dtype} and {Bs.dtype}")
    M, K = A.shape
    N, Kb = B.shape
    if K != Kb:
        raise ValueError(f"A is [M={M}, K={K}] but B is [N={N}, K={Kb}]")
    kblocks = -(-K // 128)
    if tuple(As.shape) != (M, kblocks) or tuple(Bs.shape) != (N, kblocks):
        raise ValueError(f"As must be [{M}, {kblocks}] and Bs [{N}, {kblocks}], got {tuple(As.shape)} and {tuple(Bs.shape)}")
    _require_cuda(A, "A")
    dev = A.device
    out = torch.empty((M, N), dtype=out_dtype, device=dev)
    if M == 0 or N == 0:
        return out
    lib = _lib.load()
    A_, B_ = _row_major(A, 16), _row_major(B, 16)
    As_, Bs_ = _row_major(As, 1), _row_major(Bs, 1)
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200fp8_gemm_rowscale_workspace_bytes(M, N, K))
        if ws_bytes < 0:
            _lib.check(-ws_bytes, "b200fp8_gemm_rowscale_workspace_bytes")
        ws = _workspace(dev, ws_bytes) if ws_bytes > 0 else None
        st = lib.b200fp8_gemm_rowscale(
            A_.data_ptr(), B_.data_ptr(), As_.data_ptr(), Bs_.data_ptr(), out.data_ptr(),
            M, N, K, _ld(A_), _ld(B_), _ld(As_), _ld(Bs_), _ld(out), _OUT_CODES[out_dtype],
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "b200fp8_gemm_rowscale")
    return out


def linear(x, B, Bs, out_dtype: torch.dtype, variant=None, out=None) -> torch.Tensor:
    """C = quantise(x) @ B.T in one library call (b200fp8_linear): x is bf16 [M, K] with K a
    multiple of 128; the first launch quantises it per 1x128 group straight into the layout the
    GEMM kernel reads, the GEMM follows. Bit-identical to quant_act() followed by gemm()."""
    if out_dtype not in _OUT_CODES:
        raise ValueError(f"output dtype must be torch.bfloat16 or torch.float32, got {out_dtype}")
    for name, t in (("x", x), ("B", B), ("Bs", Bs)):
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
        if t.device != x.device:
            raise ValueError("all tensors must be on the same device")
    if x.dtype != torch.bfloat16:
        raise ValueError(f"x must be torch.bfloat16, got {x.dtype}")
    if B.dtype != FP8 or Bs.dtype != torch.float32:
        raise ValueError(f"B must be torch.float8_e4m3fn and Bs torch.float32, got {B.dtype} and {Bs.dtype}")
    M, K = x.shape
    N, Kb = B.shape
    if K != Kb:
        raise ValueError(f"x is [M={M}, K={K}] but B is [N={N}, K={Kb}]")
    if K % 128 != 0:
        raise ValueError(f"K = {K} must be a multiple of 128 for the fused quantise-and-multiply call")
    kblocks, nblocks = K // 128, -(-N // 128)
    if tuple(Bs.shape) != (nblocks, kblocks):
        raise ValueError(f"Bs must be [ceil(N/128), K/128] = [{nblocks}, {kblocks}], got {tuple(Bs.shape)}")
    _require_cuda(x, "x")
    dev = x.device
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    elif tuple(out.shape) != (M, N) or out.dtype != out_dtype or out.device != dev or (N > 1 and out.stride(1) != 1):
        raise ValueError("out has the wrong shape, dtype, device or stride")
    if M == 0 or N == 0:
        return out
    lib = _lib.load()
    x_, B_, Bs_ = _row_major(x, 8), _row_major(B, 16), _row_major(Bs, 1)
    v = resolve_variant(variant)
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200fp8_linear_workspace_bytes(M, N, K, v))
        if ws_bytes < 0:
            _lib.check(-ws_bytes, "b200fp8_linear_workspace_bytes")
        ws = _workspace(dev, ws_bytes) if ws_bytes > 0 else None
        st = lib.b200fp8_linear(
            x_.data_ptr(), B_.data_ptr(), Bs_.data_ptr(), out.data_ptr(), M, N, K, _ld(x_), _ld(B_), _ld(Bs_), _ld(out),
            _OUT_CODES[out_dtype], v, ws.data_ptr() if ws is not None else None,
            ws.numel() if ws is not None else 0, status_word(dev).data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "b200fp8_linear")
    return out


def gemm_scatter(A, B, As, Bs, dst_ptrs, dst_lds, out_dtype: torch.dtype, variant=None) -> None:
    """C = A @ B.T written into several [M, >= N] buffers at once (b200fp8_gemm_scatter).
    dst_ptrs[0] / dst_lds[0] describe this GPU's own buffer, the others are device addresses of
    peer buffers mapped into this process (see PeerBuffers in tp.py); all point at the first
    element of this call's column slice.  Shapes and dtypes as for gemm(); inputs must already
    be row-major views the kernels can address."""
    import ctypes

    if out_dtype not in _OUT_CODES:
        raise ValueError(f"output dtype must be torch.bfloat16 or torch.float32, got {out_dtype}")
    _require_cuda(A, "A")
    M, K = A.shape
    N = B.shape[0]
    n = len(dst_ptrs)
    if n < 1 or n > 8 or len(dst_lds) != n:
        raise ValueError("between 1 and 8 destinations, one leading dimension each")
    if M == 0 or N == 0:
        return
    dev = A.device
    lib = _lib.load()
    A_, B_ = _row_major(A, 16), _row_major(B, 16)
    As_, Bs_ = _row_major(As, 1), _row_major(Bs, 1)
    v = resolve_variant(variant)
    ptrs = (ctypes.c_void_p * n)(*[int(p) for p in dst_ptrs])
    lds = (ctypes.c_int64 * n)(*[int(x) for x in dst_lds])
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200fp8_gemm_workspace_bytes(M, N, K, v))
        if ws_bytes < 0:
            _lib.check(-ws_bytes, "b200fp8_gemm_workspace_bytes")
        ws = _workspace(dev, ws_bytes) if ws_bytes > 0 else None
        st = lib.b200fp8_gemm_scatter(
            A_.data_ptr(), B_.data_ptr(), As_.data_ptr(), Bs_.data_ptr(), n, ptrs, lds,
            M, N, K, _ld(A_), _ld(B_), _ld(As_), _ld(Bs_), _OUT_CODES[out_dtype], v,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "b200fp8_gemm_scatter")


def gemm_multicast(A, B, As, Bs, mc_ptr: int, ldc: int, out_dtype: torch.dtype, variant=None) -> None:
    """C = A @ B.T written through a multimem (NVLink multicast) address (b200fp8_gemm_multicast):
    mc_ptr is the multicast view of a buffer that every GPU of the group holds, already offset to
    the first element of this call's column slice; ldc is the buffer's row pitch in elements.
    The NVSwitch replicates every store into all GPUs' copies (see MulticastBuffers in tp.py)."""
    if out_dtype not in _OUT_CODES:
        raise ValueError(f"output dtype must be torch.bfloat16 or torch.float32, got {out_dtype}")
    _require_cuda(A, "A")
    if not mc_ptr:
        raise ValueError("mc_ptr is null: the group has no multicast mapping")
    M, K = A.shape
    N = B.shape[0]
    if M == 0 or N == 0:
        return
    dev = A.device
    lib = _lib.load()
    A_, B_ = _row_major(A, 16), _row_major(B, 16)
    As_, Bs_ = _row_major(As, 1), _row_major(Bs, 1)
    v = resolve_variant(variant)
    with torch.cuda.device(dev):
        ws_bytes = int(lib.b200fp8_gemm_workspace_bytes(M, N, K, v))
        if ws_bytes < 0:
            _lib.check(-ws_bytes, "b200fp8_gemm_workspace_bytes")
        ws = _workspace(dev, ws_bytes) if ws_bytes > 0 else None
        st = lib.b200fp8_gemm_multicast(
            A_.data_ptr(), B_.data_ptr(), As_.data_ptr(), Bs_.data_ptr(), int(mc_ptr),
            M, N, K, _ld(A_), _ld(B_), _ld(As_), _ld(Bs_), int(ldc), _OUT_CODES[out_dtype], v,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status_word(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "b200fp8_gemm_multicast")


def _quant_common(x: torch.Tensor, name: str):
    if x.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(x.shape)}")
    if x.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be torch.bfloat16, got {x.dtype}")
    if x.shape[1] % 8 != 0:
        raise ValueError(f"K = {x.shape[1]} must be a multiple of 8")
    _require_cuda(x, name)
    return _row_major(x, 8)


def quant_act(x: torch.Tensor, group: int = 128):
    if int(group) != 128:
        raise ValueError(f"group size must be 128, got {group}")
    x_ = _quant_common(x, "x")
    M, K = x_.shape
    q = torch.empty((M, K), dtype=FP8, device=x.device)
    s = torch.empty((M, -(-K // 128)), dtype=torch.float32, device=x.device)
    if M == 0 or K == 0:
        return q, s
    with torch.cuda.device(x.device):
        st = _lib.load().b200fp8_quant_act(x_.data_ptr(), q.data_ptr(), s.data_ptr(), M, K, _ld(x_), _ld(q), _ld(s),
                                           torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(st, "b200fp8_quant_act")
    return q, s


def quant_weight(w: torch.Tensor, block: int = 128):
    if int(block) != 128:
        raise ValueError(f"block size must be 128, got {block}")
    w_ = _quant_common(w, "w")
    N, K = w_.shape
    q = torch.empty((N, K), dtype=FP8, device=w.device)
    s = torch.empty((-(-N // 128), -(-K // 128)), dtype=torch.float32, device=w.device)
    if N == 0 or K == 0:
        return q, s
    with torch.cuda.device(w.device):
        st = _lib.load().b200fp8_quant_weight(w_.data_ptr(), q.data_ptr(), s.data_ptr(), N, K, _ld(w_), _ld(q),
                                              _ld(s), torch.cuda.current_stream(w.device).cuda_stream)
    _lib.check(st, "b200fp8_quant_weight")
    return q, s
