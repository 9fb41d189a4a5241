"""Python front doors of the B200 paged latent-attention (MLA) decode path.

Same names, argument meaning and error behaviour as the reference's
``attention/mla.py`` for this path: ``mla_query_absorb`` (mla.py:17-19),
``mla_value_project`` (mla.py:22-24), ``latent_kv_write`` (mla.py:27-30),
``mla_latent_attention`` (mla.py:33-40) and ``mla_decode`` (mla.py:43-53).
Behind them ctypes calls into the C-ABI library replace the reference's
``torch.ops.qd_attention.mla_*`` dispatch.  The paged cache is
``[blocks, page, Dc+Dr]``; every input is contiguous and on one CUDA device;
page ids, positions, lengths, cache slots and selected indices are caller-owned
metadata and must be valid.  No backward.  There is no CPU fallback.
"""

from __future__ import annotations

import math

import torch

from .core import (_DTYPE_CODE, _check, _check_cuda_contiguous, _lib, _on_device, _raise_status,
                   _stream_handle)

# (device index, stream handle) -> uint8 scratch tensor of the MLA operators.  Kept apart from
# the GQA decode workspaces: those carry control words that must stay zero between calls.
_workspaces: dict[tuple[int, int], torch.Tensor] = {}

_KERNEL_CODE = {"auto": 0, "simt": 1, "tcgen05": 4}


def _same_device(base, *tensors):
    for name, t in tensors:
        _check_cuda_contiguous(t, name)
        _check(t.device == base.device, f"{name} must be contiguous and on the same CUDA device")


def _check_dtype(t):
    _check(t.dtype in _DTYPE_CODE, "dtype must be float32/float16/bfloat16")


def _scratch(device, stream, need):
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _project(x, w, absorb: bool):
    """Argument checks of mla_project_cuda (csrc/cuda/mla/mla.cu:138-146)."""
    lib = _lib()
    _check_cuda_contiguous(x, "x")
    _same_device(x, ("w", w))
    _check_dtype(x)
    _check(x.dtype == w.dtype, "dtype mismatch")
    _check(x.dim() == 4 and w.dim() == 3 and x.size(2) == w.size(0),
           "x [B,T,H,D], weight [H,Dn,Dc] or [H,Dv,Dc]")
    d_in = x.size(3)
    d_out = w.size(2) if absorb else w.size(1)
    _check(d_in > 0 and d_out > 0 and (w.size(1) == d_in if absorb else w.size(2) == d_in),
           "projection dimension mismatch")
    out = torch.empty((x.size(0), x.size(1), x.size(2), d_out), dtype=x.dtype, device=x.device)
    if out.numel() == 0:
        return out
    with _on_device(x.device):
        rc = lib.mla_b200_project(x.data_ptr(), w.data_ptr(), out.data_ptr(), _DTYPE_CODE[x.dtype],
                                  x.size(0) * x.size(1), x.size(2), d_in, d_out, 1 if absorb else 0,
                                  _stream_handle(x.device))
    _raise_status(rc, "mla_project")
    return out


def mla_query_absorb(q_nope, w_uk):
    """``q_nope [B,T,H,Dn]`` . ``w_uk [H,Dn,Dc]`` -> ``[B,T,H,Dc]``."""
    return _project(q_nope, w_uk, True)


def mla_value_project(latent_output, w_uv):
    """``latent_output [B,T,H,Dc]`` . ``w_uv [H,Dv,Dc]``^T -> ``[B,T,H,Dv]``."""
    return _project(latent_output, w_uv, False)


def latent_kv_write(latent, rope_key, cache, slot_mapping):
    """In-place write of ``latent [N,Dc]`` and ``rope_key [N,Dr]`` to unique physical int64 slots
    of ``cache [blocks, page, Dc+Dr]`` (checks of latent_kv_write_cuda, mla.cu:151-156)."""
    lib = _lib()
    _check_cuda_contiguous(latent, "latent")
    _same_device(latent, ("rope", rope_key), ("cache", cache), ("slots", slot_mapping))
    _check_dtype(latent)
    _check(latent.dim() == 2 and rope_key.dim() == 2 and cache.dim() == 3 and slot_mapping.dim() == 1
           and latent.size(0) == rope_key.size(0) and slot_mapping.size(0) == latent.size(0),
           "invalid latent/rope/cache/slots shape")
    _check(latent.size(1) > 0 and rope_key.size(1) > 0 and cache.size(1) > 0
           and cache.size(2) == latent.size(1) + rope_key.size(1), "invalid cache width")
    _check(slot_mapping.dtype == torch.int64 and latent.dtype == rope_key.dtype == cache.dtype,
           "slots must be int64 and tensors must share dtype")
    if latent.size(0) == 0:
        return
    with _on_device(latent.device):
        rc = lib.mla_b200_latent_kv_write(latent.data_ptr(), rope_key.data_ptr(), cache.data_ptr(),
                                          slot_mapping.data_ptr(), latent.size(0), latent.size(1),
                                          rope_key.size(1), _DTYPE_CODE[latent.dtype],
                                          _stream_handle(latent.device))
    _raise_status(rc, "latent_kv_write")


def _check_attend(q, qr, cache, table, lens, positions, indices, scale):
    """Argument checks of mla_attend_cuda (csrc/cuda/mla/mla.cu:162-171)."""
    _check_cuda_contiguous(q, "q")
    _same_device(q, ("q_rope", qr), ("cache", cache), ("table", table), ("lengths", lens),
                 ("positions", positions))
    _check_dtype(q)
    _check(q.dim() == 4 and qr.dim() == 4 and cache.dim() == 3 and table.dim() == 2
           and lens.dim() == 1 and positions.dim() == 2, "invalid tensor ranks")
    _check(q.shape[:3] == qr.shape[:3] and q.size(0) == table.size(0) == lens.size(0)
           and positions.size(0) == q.size(0) and positions.size(1) == q.size(1), "shape mismatch")
    _check(q.dtype == qr.dtype == cache.dtype, "dtype mismatch")
    _check(table.dtype == torch.int32 and lens.dtype == torch.int32 and positions.dtype == torch.int32,
           "metadata must be int32")
    _check(math.isfinite(scale) and scale > 0, "scale must be positive and finite")
    if indices is not None:
        _same_device(q, ("indices", indices))
        _check(indices.dim() == 3 and indices.size(0) == q.size(0) and indices.size(1) == q.size(1)
               and indices.dtype == torch.int32, "indices must be int32 [B,T,K]")


_attend_need: dict[tuple, int] = {}


def _attend_inputs_ok(q, qr, cache, table, lens, positions, indices, scale) -> bool:
    """One boolean for "every check below passes" (the common case); on False the caller runs the
    detailed checks, which raise the specific message."""
    try:
        dev, dt = q.device, q.dtype
        ok = (q.is_cuda and dt in _DTYPE_CODE and qr.dtype == dt and cache.dtype == dt
              and qr.device == dev and cache.device == dev and table.device == dev and lens.device == dev
              and positions.device == dev
              and q.is_contiguous() and qr.is_contiguous() and cache.is_contiguous() and table.is_contiguous()
              and lens.is_contiguous() and positions.is_contiguous()
              and q.dim() == 4 and qr.dim() == 4 and cache.dim() == 3 and table.dim() == 2 and lens.dim() == 1
              and positions.dim() == 2 and q.shape[:3] == qr.shape[:3]
              and q.size(0) == table.size(0) == lens.size(0) == positions.size(0) and positions.size(1) == q.size(1)
              and table.dtype == torch.int32 and lens.dtype == torch.int32 and positions.dtype == torch.int32
              and 0.0 < scale < math.inf
              and 0 < q.size(3) <= 512 and qr.size(3) > 0 and cache.size(2) == q.size(3) + qr.size(3)
              and cache.size(0) > 0 and cache.size(1) > 0 and table.size(1) > 0 and q.size(2) > 0)
        if ok and indices is not None:
            ok = (indices.is_cuda and indices.device == dev and indices.is_contiguous() and indices.dim() == 3
                  and indices.size(0) == q.size(0) and indices.size(1) == q.size(1) and indices.dtype == torch.int32)
        return bool(ok)
    except (AttributeError, TypeError):
        return False


def mla_latent_attention(q_absorbed, q_rope, cache, block_table, lengths, positions, *, scale,
                         causal=True, indices=None, kernel="auto", splits=0):
    """Latent output ``[B,T,H,Dc]``; ``indices`` are logical int32 ``[B,T,K]``.

    ``positions`` are absolute int32 ``[B,T]``.  Empty / fully masked rows return zeros.
    -1 sparse indices are ignored; all remaining indices must be unique and valid.
    ``kernel`` (``"auto" | "simt" | "tcgen05"``) and ``splits`` are tuning knobs the reference
    does not have.
    """
    lib = _lib()
    scale = float(scale)
    q = q_absorbed
    if not _attend_inputs_ok(q, q_rope, cache, block_table, lengths, positions, indices, scale):
        _check_attend(q_absorbed, q_rope, cache, block_table, lengths, positions, indices, scale)
        _check(q.size(3) > 0 and q.size(3) <= 512 and q_rope.size(3) > 0
               and cache.size(2) == q.size(3) + q_rope.size(3) and cache.size(0) > 0 and cache.size(1) > 0
               and block_table.size(1) > 0 and q.size(2) > 0, "invalid dimensions")
        raise RuntimeError("invalid mla_latent_attention arguments")   # not reached: a check above raises
    if kernel not in _KERNEL_CODE:
        raise ValueError("kernel must be auto, simt or tcgen05")
    out = torch.empty_like(q)
    if q.numel() == 0:
        return out
    nk = 0 if indices is None else indices.size(2)
    if indices is not None and nk == 0:
        return out.zero_()
    with _on_device(q.device):
        stream = _stream_handle(q.device)
        key = (q.size(0), q.size(1), q.size(2), q.size(3), q_rope.size(3), cache.size(1), block_table.size(1), nk,
               splits)
        need = _attend_need.get(key)
        if need is None:
            need = int(lib.mla_b200_attend_ex_workspace_bytes(*key[:8], int(splits)))
            _attend_need[key] = need
        ws = _scratch(q.device, stream, need)
        rc = lib.mla_b200_attend_ex(
            q.data_ptr(), q_rope.data_ptr(), cache.data_ptr(), block_table.data_ptr(), lengths.data_ptr(),
            positions.data_ptr(), None if indices is None else indices.data_ptr(), out.data_ptr(),
            _DTYPE_CODE[q.dtype], q.size(0), q.size(1), q.size(2), q.size(3), q_rope.size(3),
            cache.size(0), cache.size(1), block_table.size(1), nk, scale, 1 if causal else 0,
            ws.data_ptr(), ws.numel(), stream, _KERNEL_CODE[kernel], int(splits))
    _raise_status(rc, "mla_latent_attention")
    return out


_decode_need: dict[tuple, int] = {}


def _decode_inputs_ok(q, qr, cache, table, lens, positions, w_uk, w_uv, indices, scale) -> bool:
    """One boolean for "every check of mla_decode passes" (the common case)."""
    try:
        dev, dt = q.device, q.dtype
        dc = w_uk.size(2)
        ok = (q.is_cuda and dt in _DTYPE_CODE and qr.dtype == dt and cache.dtype == dt and w_uk.dtype == dt
              and w_uv.dtype == dt
              and all(t.device == dev and t.is_contiguous()
                      for t in (q, qr, cache, table, lens, positions, w_uk, w_uv))
              and q.dim() == 4 and qr.dim() == 4 and cache.dim() == 3 and table.dim() == 2 and lens.dim() == 1
              and positions.dim() == 2 and w_uk.dim() == 3 and w_uv.dim() == 3 and q.shape[:3] == qr.shape[:3]
              and q.size(0) == table.size(0) == lens.size(0) == positions.size(0) and positions.size(1) == q.size(1)
              and table.dtype == torch.int32 and lens.dtype == torch.int32 and positions.dtype == torch.int32
              and 0.0 < scale < math.inf
              and q.size(2) > 0 and q.size(3) > 0 and qr.size(3) > 0 and 0 < dc <= 512 and w_uv.size(1) > 0
              and w_uk.size(0) == q.size(2) and w_uk.size(1) == q.size(3) and w_uv.size(0) == q.size(2)
              and w_uv.size(2) == dc and cache.size(2) == dc + qr.size(3) and cache.size(0) > 0
              and cache.size(1) > 0 and table.size(1) > 0)
        if ok and indices is not None:
            ok = (indices.is_cuda and indices.device == dev and indices.is_contiguous() and indices.dim() == 3
                  and indices.size(0) == q.size(0) and indices.size(1) == q.size(1) and indices.dtype == torch.int32)
        return bool(ok)
    except (AttributeError, TypeError):
        return False


def mla_decode(q_nope, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, *, scale=None,
               causal=True, indices=None):
    """Absorbed paged MLA for decode or multiple queries; pre-applied RoPE.  ``[B,T,H,Dv]``.

    One C-ABI call runs query absorption, paged latent attention and the value projection
    back to back on the current stream (checks of mla_decode_fused_cuda, mla.cu:184-192).
    """
    lib = _lib()
    if scale is None:
        scale = 1.0 / math.sqrt(q_nope.shape[-1] + q_rope.shape[-1])
    scale = float(scale)
    q = q_nope
    if _decode_inputs_ok(q, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, indices, scale):
        return _mla_decode_checked(lib, q, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, scale,
                                   causal, indices)
    _check_attend(q_nope, q_rope, cache, block_table, lengths, positions, indices, scale)
    _same_device(q_nope, ("w_uk", w_uk), ("w_uv", w_uv))
    _check(w_uk.dim() == 3 and w_uv.dim() == 3, "invalid tensor ranks")
    dc = w_uk.size(2)
    _check(q.size(2) > 0 and q.size(3) > 0 and q_rope.size(3) > 0 and 0 < dc <= 512 and w_uv.size(1) > 0
           and w_uk.size(0) == q.size(2) and w_uk.size(1) == q.size(3) and w_uv.size(0) == q.size(2)
           and w_uv.size(2) == dc and cache.size(2) == dc + q_rope.size(3) and cache.size(0) > 0
           and cache.size(1) > 0 and block_table.size(1) > 0, "invalid dimensions")
    _check(q.dtype == w_uk.dtype == w_uv.dtype, "dtype mismatch")
    raise RuntimeError("invalid mla_decode arguments")   # not reached: a check above raises


def _mla_decode_checked(lib, q, q_rope, cache, block_table, lengths, positions, w_uk, w_uv, scale, causal,
                        indices):
    dc = w_uk.size(2)
    out = torch.empty((q.size(0), q.size(1), q.size(2), w_uv.size(1)), dtype=q.dtype, device=q.device)
    if out.numel() == 0:
        return out
    nk = 0 if indices is None else indices.size(2)
    if indices is not None and nk == 0:
        return out.zero_()
    with _on_device(q.device):
        stream = _stream_handle(q.device)
        key = (q.size(0), q.size(1), q.size(2), dc, q_rope.size(3), cache.size(1), block_table.size(1), nk)
        need = _decode_need.get(key)
        if need is None:
            need = _decode_need[key] = int(lib.mla_b200_decode_workspace_bytes(*key))
        ws = _scratch(q.device, stream, need)
        rc = lib.mla_b200_decode(
            q.data_ptr(), q_rope.data_ptr(), cache.data_ptr(), block_table.data_ptr(), lengths.data_ptr(),
            positions.data_ptr(), w_uk.data_ptr(), w_uv.data_ptr(),
            None if indices is None else indices.data_ptr(), out.data_ptr(), _DTYPE_CODE[q.dtype],
            q.size(0), q.size(1), q.size(2), q.size(3), q_rope.size(3), dc, w_uv.size(1), cache.size(0),
            cache.size(1), block_table.size(1), nk, scale, 1 if causal else 0, ws.data_ptr(), ws.numel(),
            stream)
    _raise_status(rc, "mla_decode")
    return out


def mla_tc_status(reset: bool = False) -> int:
    """Status word of the tensor-core attention kernel's bounded waits on the current device
    (0 = no wait ever ran out).  Synchronises the device."""
    return int(_lib().mla_b200_tc_status(1 if reset else 0))
