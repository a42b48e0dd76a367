"""PyTorch-facing wrappers of the decode-step glue kernels (`csrc/decoder_glue.cu`):
residual add + RMSNorm, rotary embedding + KV-cache write, single-query attention over
the cache, and SwiGLU's `silu(gate) * up`.  bf16 CUDA tensors only; launches go to the
current stream and record into CUDA graphs."""

from __future__ import annotations

import torch

from . import _lib


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _bf16(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise RuntimeError("glue kernels take contiguous bf16 CUDA tensors")


def _positions(positions: torch.Tensor, batch: int, device: torch.device) -> None:
    """Positions are read on the device as int64: anything else would be misread."""
    if (not positions.is_cuda or positions.device != device or positions.dtype != torch.int64
            or not positions.is_contiguous() or positions.numel() != batch):
        raise ValueError(f"positions must be a contiguous int64 tensor of {batch} entries on {device}, not "
                         f"{positions.dtype}{list(positions.shape)} on {positions.device}")


def decoder_status() -> None:
    """Raises if a decode-step kernel met a position outside its cache since the last call
    (synchronises the device; `b200q_decoder_status`)."""
    _lib.check(_lib.load().b200q_decoder_status())


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """`x += delta` in place (when given), returns `rms_norm(x) * weight`."""
    _bf16(x, weight, *([] if delta is None else [delta]))
    rows, hidden = x.shape
    y = torch.empty_like(x)
    _lib.check(_lib.load().b200q_add_rmsnorm(x.data_ptr(), None if delta is None else delta.data_ptr(),
                                             weight.data_ptr(), y.data_ptr(), rows, hidden, eps, _stream(x)))
    return y


def rope_cache(qkv: torch.Tensor, positions: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
               nq: int, nkv: int, theta: float) -> torch.Tensor:
    """Rotates q and k of `qkv` [B, (nq + 2 nkv) * D], writes k and v into the caches
    [B, nkv, S, D] at `positions` and returns q [B, nq, D]."""
    _bf16(qkv, cache_k, cache_v)
    batch = qkv.shape[0]
    _positions(positions, batch, qkv.device)
    _, _, max_seq, hd = cache_k.shape
    q = torch.empty(batch, nq, hd, device=qkv.device, dtype=qkv.dtype)
    _lib.check(_lib.load().b200q_rope_cache(qkv.data_ptr(), positions.data_ptr(), q.data_ptr(),
                                            cache_k.data_ptr(), cache_v.data_ptr(), batch, nq, nkv, hd,
                                            max_seq, theta, _stream(qkv)))
    return q


def attention_splits(batch: int, nkv: int, max_seq: int, sms: int = 148) -> int:
    """Key splits (a power of two, at least 64 positions each) for about two blocks per
    multiprocessor: measured on a B200 at 2048 positions, batch 1 is fastest with 8 splits,
    batch 8 with 4, batch 64 with 1."""
    want = max(1, (2 * sms) // max(1, batch * nkv))
    splits = 1
    while splits * 2 <= want and max_seq // (splits * 2) >= 64:
        splits *= 2
    return splits


def decode_attention(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
                     positions: torch.Tensor, splits: int | None = None) -> torch.Tensor:
    """Attention of one query per row, q [B, nq, D], over cache positions 0..positions[b];
    returns [B, nq * D].  Up to 8 key splits run as one launch (the splits of a row and KV
    head are a thread-block cluster); more need a scratch tensor and a second, merging launch."""
    _bf16(q, cache_k, cache_v)
    batch, nq, hd = q.shape
    _positions(positions, batch, q.device)
    _, nkv, max_seq, _ = cache_k.shape
    if splits is None:
        splits = min(8, attention_splits(batch, nkv, max_seq))
    lib = _lib.load()
    out = torch.empty(batch, nq * hd, device=q.device, dtype=q.dtype)
    if splits <= 8:
        _lib.check(lib.b200q_decode_attention_cluster(q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                                                      positions.data_ptr(), out.data_ptr(), batch, nq, nkv, hd,
                                                      max_seq, splits, _stream(q)))
        return out
    scratch = torch.empty(lib.b200q_decode_attention_scratch_bytes(batch, nq, hd, splits), dtype=torch.uint8,
                          device=q.device)
    _lib.check(lib.b200q_decode_attention(q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                                          positions.data_ptr(), out.data_ptr(), scratch.data_ptr(), batch, nq,
                                          nkv, hd, max_seq, splits, _stream(q)))
    return out


def rope_table(max_seq: int, head_dim: int, theta: float, device: torch.device) -> torch.Tensor:
    """(cos, sin) of every position and frequency, f32 [max_seq, head_dim / 2, 2], for `rope_attention`."""
    table = torch.empty(max_seq, head_dim // 2, 2, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(_lib.load().b200q_rope_table(table.data_ptr(), max_seq, head_dim, float(theta),
                                                torch.cuda.current_stream(device).cuda_stream))
    return table


def rope_attention(qkv: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, cache_k: torch.Tensor,
                   cache_v: torch.Tensor, nq: int, nkv: int, splits: int | None = None) -> torch.Tensor:
    """`rope_cache` + `decode_attention` in one launch: rotates q and k of the fused projection
    qkv [B, (nq + 2 nkv) * D] at positions[b], appends k and v to the caches and attends over
    positions 0..positions[b]; returns [B, nq * D]."""
    _bf16(qkv, cache_k, cache_v)
    batch, _, max_seq, hd = cache_k.shape
    _positions(positions, batch, qkv.device)
    if splits is None:
        splits = min(8, attention_splits(batch, nkv, max_seq))
    if table.shape != (max_seq, hd // 2, 2) or table.dtype != torch.float32:
        raise ValueError("rope_attention: the table does not match the cache")
    out = torch.empty(batch, nq * hd, device=qkv.device, dtype=qkv.dtype)
    _lib.check(_lib.load().b200q_rope_attention(qkv.data_ptr(), positions.data_ptr(), table.data_ptr(),
                                                cache_k.data_ptr(), cache_v.data_ptr(), out.data_ptr(), batch, nq,
                                                nkv, hd, max_seq, splits, _stream(qkv)))
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """`silu(gate_up[:, :I]) * gate_up[:, I:]` for gate_up [B, 2 I]."""
    _bf16(gate_up)
    rows, width = gate_up.shape
    out = torch.empty(rows, width // 2, device=gate_up.device, dtype=gate_up.dtype)
    _lib.check(_lib.load().b200q_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, width // 2, _stream(gate_up)))
    return out
