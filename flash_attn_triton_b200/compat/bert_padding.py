"""Un-padding and re-padding of a batch around variable-length attention.

Same functions as the reference's flash_attn/bert_padding.py (index_first_axis :8-35,
index_put_first_axis :41-64, index_first_axis_residual :70-95, unpad_input :98-122,
unpad_input_for_concatenated_sequences :125-194, pad_input :197-213).  The row gathers and
scatters -- the part that moves the hidden states -- are CUDA kernels behind the C ABI
(fa_gather_rows / fa_scatter_rows); index bookkeeping (nonzero, cumsum) stays in torch.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _native as N

_DT = {torch.float16: N.FA_F16, torch.bfloat16: N.FA_BF16, torch.float32: N.FA_F32}


def _rows(t):
    """(rows, row_bytes) of `t` seen as a matrix over its first axis, or None when the row movers
    cannot take it (rows not a multiple of 16 bytes / not 16-byte aligned / not CUDA)."""
    if not t.is_cuda or t.ndim < 2 or not t.is_contiguous():
        return None
    row_bytes = (t.numel() // max(t.shape[0], 1)) * t.element_size() if t.shape[0] else 0
    if t.shape[0] and (row_bytes % 16 or t.data_ptr() % 16):
        return None
    return t.shape[0], row_bytes


def _gather(src, idx):
    idx = idx.to(device=src.device, dtype=torch.int64).contiguous()
    src = src.contiguous()
    out = torch.empty((idx.numel(),) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    r = _rows(src)
    if r is None or _rows(out) is None:
        raise ValueError("index_first_axis needs CUDA tensors whose rows are 16-byte multiples")
    if idx.numel():
        dev = src.device.index if src.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(src.device):
            N.check(N.lib().fa_gather_rows(src.data_ptr(), out.data_ptr(), idx.data_ptr(), idx.numel(),
                                           r[1], r[0], dev, N.stream_ptr(src.device)), "fa_gather_rows")
    return out


def _scatter(src, idx, out, add):
    """out[idx[i]] = src[i] (add=False) or += (add=True); idx distinct."""
    idx = idx.to(device=src.device, dtype=torch.int64).contiguous()
    src = src.contiguous()
    r = _rows(out)
    if r is None or _rows(src) is None:
        raise ValueError("index_put_first_axis needs CUDA tensors whose rows are 16-byte multiples")
    if idx.numel():
        dev = src.device.index if src.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(src.device):
            N.check(N.lib().fa_scatter_rows(src.data_ptr(), out.data_ptr(), idx.data_ptr(), idx.numel(),
                                            r[1], r[0], _DT[src.dtype] if add else -1, dev,
                                            N.stream_ptr(src.device)), "fa_scatter_rows")
    return out


def _check_dtype(t):
    if t.dtype not in _DT:
        raise ValueError("supported dtypes: float16, bfloat16, float32")


class IndexFirstAxis(torch.autograd.Function):
    """out = input[indices] over the first axis; the gradient scatters into zeros."""

    @staticmethod
    def forward(ctx, input, indices):
        assert input.ndim >= 2
        _check_dtype(input)
        ctx.save_for_backward(indices)
        ctx.first_axis_dim = input.shape[0]
        return _gather(input, indices)

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        grad_input = torch.zeros((ctx.first_axis_dim,) + tuple(grad_output.shape[1:]),
                                 device=grad_output.device, dtype=grad_output.dtype)
        _scatter(grad_output, indices, grad_input, add=False)
        return grad_input, None


index_first_axis = IndexFirstAxis.apply


class IndexPutFirstAxis(torch.autograd.Function):
    """Zeros of first_axis_dim rows with values written at `indices`; the gradient gathers."""

    @staticmethod
    def forward(ctx, values, indices, first_axis_dim):
        assert indices.ndim == 1 and values.ndim >= 2
        _check_dtype(values)
        ctx.save_for_backward(indices)
        output = torch.zeros((first_axis_dim,) + tuple(values.shape[1:]), device=values.device,
                             dtype=values.dtype)
        return _scatter(values, indices, output, add=False)

    @staticmethod
    def backward(ctx, grad_output):
        (indices,) = ctx.saved_tensors
        return _gather(grad_output, indices), None, None


index_put_first_axis = IndexPutFirstAxis.apply


class IndexFirstAxisResidual(torch.autograd.Function):
    """Returns (input[indices], input); the gradient is grad_residual with grad_output added
    at `indices` (in place, like the reference's scatter_add_)."""

    @staticmethod
    def forward(ctx, input, indices):
        assert input.ndim >= 2
        _check_dtype(input)
        ctx.save_for_backward(indices)
        ctx.first_axis_dim = input.shape[0]
        return _gather(input, indices), input.detach()

    @staticmethod
    def backward(ctx, grad_output, grad_residual):
        (indices,) = ctx.saved_tensors
        assert grad_residual.shape[1:] == grad_output.shape[1:]
        grad_input = grad_residual.contiguous()
        _scatter(grad_output, indices, grad_input, add=True)
        return grad_input.reshape((ctx.first_axis_dim,) + tuple(grad_output.shape[1:])), None


index_first_axis_residual = IndexFirstAxisResidual.apply


def unpad_input(hidden_states, attention_mask):
    """hidden_states (batch, seqlen, ...), attention_mask (batch, seqlen) with 1 = valid ->
    (tokens (total_nnz, ...), indices (total_nnz,), cu_seqlens (batch + 1,) int32, max_seqlen)."""
    seqlens_in_batch = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    max_seqlen_in_batch = seqlens_in_batch.max().item()
    cu_seqlens = F.pad(torch.cumsum(seqlens_in_batch, dim=0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape((-1,) + tuple(hidden_states.shape[2:]))
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen_in_batch


def unpad_input_for_concatenated_sequences(hidden_states, attention_mask_in_length):
    """Like unpad_input for rows that hold several short samples back to back:
    attention_mask_in_length[b] lists the lengths of the samples of row b, zero-padded."""
    length = attention_mask_in_length.sum(dim=-1)
    seqlen = attention_mask_in_length.size(-1)
    attention_mask_2d = torch.arange(seqlen, device=length.device, dtype=length.dtype).expand(
        len(length), seqlen) < length.unsqueeze(1)
    real_indices_idx = torch.nonzero(attention_mask_in_length.flatten(), as_tuple=False).flatten()
    seqlens_in_batch = attention_mask_in_length.flatten()[real_indices_idx]
    indices = torch.nonzero(attention_mask_2d.flatten(), as_tuple=False).flatten()
    max_seqlen_in_batch = seqlens_in_batch.max().item()
    cu_seqlens = F.pad(torch.cumsum(seqlens_in_batch, dim=0, dtype=torch.int32), (1, 0))
    flat = hidden_states.reshape((-1,) + tuple(hidden_states.shape[2:]))
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen_in_batch


def pad_input(hidden_states, indices, batch, seqlen):
    """tokens (total_nnz, ...) -> (batch, seqlen, ...) with zeros at the padded positions."""
    output = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return output.reshape((batch, seqlen) + tuple(hidden_states.shape[1:]))
