"""Python front doors of the B200 paged GQA decode path.

Same names, argument meaning and error behaviour as the reference's
``attention/core.py`` for this path: ``gqa_decode`` (core.py:17-40),
``gqa_decode_split`` (core.py:43-56), ``gqa_decode_auto`` (core.py:80-96),
``kv_append`` (core.py:59-63) and ``is_cuda_extension_loaded`` (core.py:13-14).
Behind them a ctypes call into the C-ABI library replaces the reference's
``torch.ops.qd_attention.*`` dispatch; torch is used here for device memory and
the current stream only.  There is no CPU fallback: without the library every
operator raises RuntimeError.
"""

from __future__ import annotations

import math
import weakref

import torch

from . import _cabi

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_KERNEL_CODE = {"auto": 0, "simt": 1, "mma": 2, "tcgen05": 4}

# (device index, stream handle) -> uint8 scratch tensor, grown on demand
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def is_cuda_extension_loaded() -> bool:
    """True when the C-ABI library (the CUDA kernels) could be loaded."""
    return _cabi.load_error() is None


def _lib():
    err = _cabi.load_error()
    if err is not None:
        raise RuntimeError(
            "gqa_decode_b200 CUDA library was not loaded. Build it with "
            "`python -m attention_b200.build` on a machine with nvcc (sm_100a)."
        ) from err
    return _cabi.load()


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda_contiguous(t: torch.Tensor, name: str) -> None:
    _check(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _validate_decode(q, k_cache, v_cache, block_table, context_lens, scale, splits=1):
    """Every argument check of gqa_decode_impl (csrc/cuda/dense/gqa_decode.cu:103-138)."""
    _check(1 <= splits <= 65535, "splits must be in [1, 65535]")
    for t, name in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache"),
                    (block_table, "block_table"), (context_lens, "context_lens")):
        _check_cuda_contiguous(t, name)
    _check(q.dim() == 3, "q must be [B, Hq, D]")
    _check(k_cache.dim() == 4, "k_cache must be [Nblocks, BlockSize, Hkv, D]")
    _check(v_cache.shape == k_cache.shape, "v_cache shape mismatch")
    _check(block_table.dim() == 2, "block_table must be [B, MaxPages]")
    _check(context_lens.dim() == 1, "context_lens must be [B]")
    _check(all(t.device == q.device for t in (k_cache, v_cache, block_table, context_lens)),
           "all tensors must use one CUDA device")
    _check(q.dtype == k_cache.dtype == v_cache.dtype, "q/k/v dtype must match")
    _check(q.dtype in _DTYPE_CODE, "q/k/v must be float32/float16/bfloat16")
    _check(block_table.dtype == torch.int32 and context_lens.dtype == torch.int32,
           "block_table and context_lens must be int32")
    _check(q.size(0) == block_table.size(0) == context_lens.size(0), "batch sizes must match")
    _check(q.size(2) == k_cache.size(3), "q head_dim and cache head_dim must match")
    _check(q.size(1) > 0 and k_cache.size(2) > 0 and q.size(1) % k_cache.size(2) == 0,
           "Hq must be divisible by Hkv")
    _check(0 < q.size(2) <= 256, "supported head_dim is [1, 256]")
    _check(k_cache.size(0) > 0 and k_cache.size(1) > 0,
           "cache must have positive blocks and block_size")
    _check(block_table.size(1) > 0, "block_table must have at least one page")
    _check(math.isfinite(scale) and scale > 0.0, "scale must be positive and finite")
    imax = 2**31 - 1
    _check(max(q.size(0), q.size(1), k_cache.size(2), k_cache.size(1), block_table.size(1),
               k_cache.size(0)) <= imax, "tensor sizes exceed int32 CUDA launch limits")


def _raise_status(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {_cabi.strerror(rc)} (status {rc})")


try:   # raw handle of the current stream without building a Stream object (a few us less)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:   # pragma: no cover - older/newer torch without the private hook
    _raw_stream = None


def _stream_handle(device: torch.device) -> int:
    if _raw_stream is not None:
        return int(_raw_stream(device.index))
    return int(torch.cuda.current_stream(device).cuda_stream)


class _on_device:
    """``with _on_device(dev):`` makes ``dev`` current only if it is not already."""

    __slots__ = ("_ctx",)

    def __init__(self, device: torch.device):
        self._ctx = None if torch.cuda.current_device() == device.index else torch.cuda.device(device)

    def __enter__(self):
        if self._ctx is not None:
            self._ctx.__enter__()

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)


def _decode_inputs_ok(q, k_cache, v_cache, block_table, context_lens, scale) -> bool:
    """One boolean for "every check of _validate_decode passes" (the common case); on False
    the caller runs _validate_decode, which raises the specific message."""
    try:
        dt = q.dtype
        dev = q.device
        return (q.is_cuda and k_cache.is_cuda and v_cache.is_cuda and block_table.is_cuda
                and context_lens.is_cuda
                and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
                and block_table.is_contiguous() and context_lens.is_contiguous()
                and q.dim() == 3 and k_cache.dim() == 4 and v_cache.shape == k_cache.shape
                and block_table.dim() == 2 and context_lens.dim() == 1
                and k_cache.device == dev and v_cache.device == dev
                and block_table.device == dev and context_lens.device == dev
                and k_cache.dtype == dt and v_cache.dtype == dt and dt in _DTYPE_CODE
                and block_table.dtype == torch.int32 and context_lens.dtype == torch.int32
                and q.size(0) == block_table.size(0) == context_lens.size(0)
                and q.size(2) == k_cache.size(3) and q.size(1) > 0 and k_cache.size(2) > 0
                and q.size(1) % k_cache.size(2) == 0 and 0 < q.size(2) <= 256
                and k_cache.size(0) > 0 and k_cache.size(1) > 0 and block_table.size(1) > 0
                and 0.0 < scale < math.inf
                and max(q.size(0), q.size(1), k_cache.size(0), k_cache.size(1),
                        block_table.size(1)) <= 2**31 - 1)
    except (AttributeError, TypeError):
        return False


_ws_need: dict[tuple, int] = {}

# Argument sets that passed every check, keyed by the identities of the five tensors: a decode
# loop calls with the same tensor objects step after step, and re-deriving ~45 properties of
# them costs more host time than a small batch takes on the GPU.  An entry is trusted only
# while all five objects are alive, identical and still at the same device addresses.
_checked: dict[tuple, tuple] = {}
_CHECKED_MAX = 256


def _checked_entry(q, k_cache, v_cache, block_table, context_lens, scale):
    key = (id(q), id(k_cache), id(v_cache), id(block_table), id(context_lens), scale)
    ent = _checked.get(key)
    if ent is not None:
        refs, ptrs = ent[0], ent[1]
        if (refs[0]() is q and refs[1]() is k_cache and refs[2]() is v_cache
                and refs[3]() is block_table and refs[4]() is context_lens
                and ptrs == (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                             block_table.data_ptr(), context_lens.data_ptr())):
            return ent
    if not _decode_inputs_ok(q, k_cache, v_cache, block_table, context_lens, scale):
        _validate_decode(q, k_cache, v_cache, block_table, context_lens, scale)
        raise RuntimeError("invalid gqa_decode arguments")   # not reached: the line above raises
    ent = (tuple(weakref.ref(t) for t in (q, k_cache, v_cache, block_table, context_lens)),
           (q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
            context_lens.data_ptr()),
           # the launcher's integer arguments, in its order
           (_DTYPE_CODE[q.dtype], q.size(0), q.size(1), k_cache.size(2), q.size(2), k_cache.size(0),
            k_cache.size(1), block_table.size(1)))
    if len(_checked) >= _CHECKED_MAX:
        _checked.clear()
    _checked[key] = ent
    return ent


def _workspace_for(lib, device, shape_key, stream):
    """shape_key = (batch, q_heads, kv_heads, head_dim, block_size, max_pages, chunk_tokens)"""
    need = _ws_need.get(shape_key)
    if need is None:
        need = int(lib.gqa_b200_workspace_bytes(*shape_key))
        _ws_need[shape_key] = need
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        # zero-filled: the control words at the start of a workspace must be zero before its
        # first call; every call leaves them at zero again
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws, need


def workspace_bytes(batch, q_heads, kv_heads, head_dim, block_size, max_pages, chunk_tokens=0) -> int:
    """Bytes of scratch ``gqa_decode`` needs for this static shape (worst case over lengths)."""
    return int(_lib().gqa_b200_workspace_bytes(batch, q_heads, kv_heads, head_dim, block_size,
                                               max_pages, chunk_tokens))


def gqa_decode(q, k_cache, v_cache, block_table, context_lens, *, scale=None, out=None,
               workspace=None, chunk_tokens=0, kernel="auto", max_ctas=0, phases=0):
    """Paged single-token MHA/MQA/GQA decode on B200.

    Inputs are CUDA and contiguous; q/k/v share a dtype (float32/float16/bfloat16).
    ``q [B,Hq,D]``, caches ``[blocks, block_size, Hkv, D]``, ``block_table [B,max_pages]``
    int32, ``context_lens [B]`` int32.  Returns ``[B,Hq,D]`` in ``q.dtype``.  Never reads
    ``context_lens`` on the host and never synchronises.  No autograd support.

    Keyword extras that the reference does not have: ``out`` (preallocated result),
    ``workspace`` (uint8 CUDA tensor of at least ``workspace_bytes(...)`` bytes, 256-byte
    aligned, **zero-filled when first used** -- ``torch.zeros`` -- after which every call
    leaves its control words at zero again; by default one is cached per device and stream),
    ``chunk_tokens`` / ``kernel`` (``"auto" | "simt" | "mma"``) / ``max_ctas`` / ``phases``
    (tuning knobs used by tests and benchmarks; ``phases`` 0 = the default single launch,
    otherwise the bit mask 1 = plan, 2 = decode, 4 = merge of the three-launch path).
    """
    lib = _lib()
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scale = float(scale)
    _, ptrs, dims = _checked_entry(q, k_cache, v_cache, block_table, context_lens, scale)
    if kernel not in ("auto", "simt", "mma"):
        raise ValueError("kernel must be auto, simt or mma")
    if out is None:
        out = torch.empty_like(q)
    else:
        _check_cuda_contiguous(out, "out")
        _check(out.shape == q.shape and out.dtype == q.dtype and out.device == q.device,
               "out must match q")
    if dims[1] == 0:
        return out
    device = q.device
    with _on_device(device):
        stream = _stream_handle(device)
        if workspace is None:
            workspace, need = _workspace_for(
                lib, device, (dims[1], dims[2], dims[3], dims[4], dims[6], dims[7], chunk_tokens), stream)
        else:
            _check(workspace.is_cuda and workspace.device == device and
                   workspace.is_contiguous() and workspace.dtype == torch.uint8,
                   "workspace must be a contiguous uint8 tensor on q's device")
        rc = lib.gqa_b200_decode_ex(
            ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], out.data_ptr(), dims[0], dims[1], dims[2],
            dims[3], dims[4], dims[5], dims[6], dims[7], scale, workspace.data_ptr(),
            workspace.numel(), stream, int(chunk_tokens), _KERNEL_CODE[kernel], int(max_ctas),
            int(phases))
    _raise_status(rc, "gqa_decode")
    return out


def gqa_decode_split(q, k_cache, v_cache, block_table, context_lens, *, splits=4, scale=None,
                     workspace=None, backend="cuda"):
    """Decode ``splits`` independent KV partitions and merge their fp32 softmax states.

    Partition z of a sequence of length L covers tokens [L*z//splits, L*(z+1)//splits);
    ``workspace`` (optional) is float32 ``[B, Hq, splits, D+2]`` = ``[max, sum, acc...]`` per
    partition, overwritten in place, and requires ``splits > 1`` -- all as in the reference
    (csrc/cuda/dense/gqa_decode.cu:40-41,67-69,148-152).  This build has no Triton backend:
    ``backend`` must be ``"cuda"``.
    """
    if backend != "cuda":
        raise ValueError("backend must be cuda (this build has no triton backend)")
    lib = _lib()
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scale = float(scale)
    splits = int(splits)
    _validate_decode(q, k_cache, v_cache, block_table, context_lens, scale, splits)
    shape = (q.size(0), q.size(1), splits, q.size(2) + 2)
    if workspace is not None:
        _check(splits > 1, "workspace requires splits > 1")
        _check(workspace.is_cuda and workspace.device == q.device and workspace.is_contiguous()
               and workspace.dtype == torch.float32,
               "workspace must be contiguous float32 on q device")
        _check(tuple(workspace.shape) == shape, "workspace shape must be [B,Hq,splits,D+2]")
    elif splits > 1:
        workspace = torch.empty(shape, dtype=torch.float32, device=q.device)
    out = torch.empty_like(q)
    if q.size(0) == 0:
        return out
    with _on_device(q.device):
        rc = lib.gqa_b200_decode_split(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
            context_lens.data_ptr(), out.data_ptr(), _DTYPE_CODE[q.dtype], q.size(0), q.size(1),
            k_cache.size(2), q.size(2), k_cache.size(0), k_cache.size(1), block_table.size(1),
            scale, splits, workspace.data_ptr() if workspace is not None else None,
            _stream_handle(q.device))
    _raise_status(rc, "gqa_decode_split")
    return out


def gqa_decode_auto(q, k_cache, v_cache, block_table, context_lens, *, scale=None):
    """Decode with the split chosen for the caller, without reading lengths on the host.

    The reference picks a split count from the static table capacity and the SM count and
    hands over to its Triton kernel (core.py:80-96).  Here ``gqa_decode`` already cuts every
    sequence into KV chunks from its own device-side length, so this is the same call.
    """
    if q.ndim != 3 or k_cache.ndim != 4 or block_table.ndim != 2:
        raise ValueError("invalid decode input dimensions")
    return gqa_decode(q, k_cache, v_cache, block_table, context_lens, scale=scale)


def kv_append(key, value, k_cache, v_cache, block_table, positions):
    """Write one token per sequence into its page; the caller owns valid, distinct
    destinations.  Checks follow kv_append_cuda (csrc/cuda/cache/kv_append.cu:32-43)."""
    lib = _lib()
    for t in (key, value, k_cache, v_cache, block_table, positions):
        _check(isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous(),
               "all tensors must be contiguous CUDA tensors")
        _check(t.device == key.device, "all tensors must share a device")
    _check(key.dim() == 3 and value.shape == key.shape, "key/value must be [B, Hkv, D]")
    _check(k_cache.dim() == 4 and v_cache.shape == k_cache.shape, "cache must be [Nblocks, P, Hkv, D]")
    _check(key.size(1) == k_cache.size(2) and key.size(2) == k_cache.size(3),
           "cache head shape mismatch")
    _check(k_cache.size(0) > 0 and k_cache.size(1) > 0 and key.size(1) > 0 and key.size(2) > 0,
           "invalid dimensions")
    _check(block_table.dim() == 2 and block_table.size(0) == key.size(0) and block_table.size(1) > 0
           and positions.dim() == 1 and positions.size(0) == key.size(0), "invalid metadata shape")
    _check(block_table.dtype == torch.int32 and positions.dtype == torch.int32,
           "metadata must be int32")
    _check(key.dtype == value.dtype == k_cache.dtype == v_cache.dtype, "dtype mismatch")
    _check(key.dtype in _DTYPE_CODE, "unsupported dtype")
    if key.size(0) == 0:
        return
    with _on_device(key.device):
        rc = lib.gqa_b200_kv_append(
            key.data_ptr(), value.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            block_table.data_ptr(), positions.data_ptr(), _DTYPE_CODE[key.dtype], key.size(0),
            key.size(1), key.size(2), k_cache.size(0), k_cache.size(1), block_table.size(1),
            _stream_handle(key.device))
    _raise_status(rc, "kv_append")


def gqa_prefill(q, k, v, q_lens, kv_lens, *, causal=True, scale=None, backend="cuda", kernel="auto"):
    """Dense ``[B,T,H,D]`` GQA prefill; causal queries align to the right of the valid KV.

    Same contract as the reference's ``gqa_prefill`` (attention/core.py:66-77,
    csrc/cuda/dense/gqa_prefill.cu:104-123): rows at or past ``q_lens[b]`` come back as zeros.
    ``backend`` is ``"cuda"`` or ``"tensorcore"`` as in the reference; both run this library's
    kernels (the tensor-core kernel is picked whenever the tensors allow it), ``"tensorcore"``
    additionally insists on fp16/bf16 like the reference's Triton path.  ``kernel`` is a
    tuning knob: ``"auto" | "simt" | "mma" | "tcgen05"``.
    """
    if backend not in ("cuda", "tensorcore"):
        raise ValueError("backend must be cuda or tensorcore")
    lib = _lib()
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scale = float(scale)
    for t in (q, k, v, q_lens, kv_lens):
        _check(isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous(),
               "all inputs must be contiguous CUDA tensors")
        _check(t.device == q.device, "all inputs must be on the same device")
    _check(q.dim() == 4 and k.dim() == 4 and v.shape == k.shape, "q/k/v must be [B,T,H,D]")
    _check(q.size(0) == k.size(0) and q.size(3) == k.size(3), "batch or head_dim mismatch")
    _check(q.size(2) > 0 and k.size(2) > 0 and q.size(2) % k.size(2) == 0, "invalid head mapping")
    _check(0 < q.size(3) <= 256, "head_dim must be in [1,256]")
    _check(q.size(0) <= 65535 and q.size(1) <= 65535 and k.size(1) <= 2**31 - 1,
           "dimensions exceed launch limits")
    _check(q_lens.dim() == 1 and kv_lens.dim() == 1 and q_lens.size(0) == q.size(0)
           and kv_lens.size(0) == q.size(0), "lengths must be [B]")
    _check(q_lens.dtype == torch.int32 and kv_lens.dtype == torch.int32, "lengths must be int32")
    _check(q.dtype == k.dtype == v.dtype, "dtype mismatch")
    _check(q.dtype in _DTYPE_CODE, "unsupported dtype")
    _check(math.isfinite(scale) and scale > 0, "scale must be positive and finite")
    if backend == "tensorcore" and q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("tensorcore backend requires matching fp16 or bf16")
    if kernel not in ("auto", "simt", "mma", "tcgen05"):
        raise ValueError("kernel must be auto, simt, mma or tcgen05")
    out = torch.empty_like(q)
    if q.size(0) == 0 or q.size(1) == 0:
        return out
    with _on_device(q.device):
        rc = lib.gqa_b200_prefill(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), q_lens.data_ptr(), kv_lens.data_ptr(),
            out.data_ptr(), _DTYPE_CODE[q.dtype], q.size(0), q.size(1), k.size(1), q.size(2),
            k.size(2), q.size(3), scale, 1 if causal else 0, _KERNEL_CODE[kernel],
            _stream_handle(q.device))
    _raise_status(rc, "gqa_prefill")
    return out
