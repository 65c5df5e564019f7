"""The sampler of a generation call: logits on the device in, token ids on the device out."""
from __future__ import annotations

from ctypes import c_float, c_int, c_ulonglong, c_void_p

import numpy as np
import torch

from ..kernels import ops
from .params import HISTORY_WINDOW, SamplingParams


_needs: dict[int, bool] = {}


def needs_scratch(V: int) -> bool:
    """Whether the sampler wants a scratch row for every row of logits: only for vocabularies too large for the
    shared memory of a thread-block cluster (the kernel that holds a row there reads the logits once)."""
    if V not in _needs:
        fn = ops._fn("sampling", "lq_sample_needs_scratch", [c_int])
        _needs[V] = bool(fn(V))
    return _needs[V]


def sample(logits: torch.Tensor, params: SamplingParams, seed: int, sequence_ids=None, steps=None,
           history: torch.Tensor | None = None, history_len: torch.Tensor | None = None,
           scratch: torch.Tensor | None = None, out: torch.Tensor | None = None, step_offset: int = 0,
           one_block: bool = False) -> torch.Tensor:
    """One token for each row of logits [rows, vocab] (float32).

    sequence_ids, steps  int32 [rows]: the counter of each row's random draw; step_offset is added to every
                         row's step (rows that advance together keep one array and pass the step here)
    one_block            run the kernel that takes a row per block with its weights in a scratch row in global
                         memory, whatever the vocabulary (by default only vocabularies too large for a cluster's
                         shared memory take it)
    history, history_len int32 [rows, 64] and [rows]: the last tokens of each sequence
    """
    rows, V = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise ops.KernelError("sample: logits must be contiguous float32")
    if scratch is None and (one_block or needs_scratch(V)):
        scratch = torch.empty((rows, V), dtype=torch.float32, device=logits.device)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if not params.greedy and (sequence_ids is None or steps is None):
        raise ops.KernelError("sample: a random draw needs sequence ids and steps")
    use_hist = params.uses_history and history is not None
    fn = ops._fn("sampling", "lq_sample_one_block" if one_block else "lq_sample", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_float, c_float,
                                           c_void_p, c_int, c_void_p, c_ulonglong, c_void_p, c_void_p, c_int, c_void_p])
    ops._check(fn(ops._p(logits), ops._p(scratch), ops._p(out), rows, V, float(params.temperature), int(params.top_k),
                  float(params.top_p), float(params.repetition_penalty),
                  ops._p(history if use_hist else None), history.stride(0) if use_hist else 0,
                  ops._p(history_len if use_hist else None), c_ulonglong(seed & 0xFFFF_FFFF_FFFF_FFFF),
                  ops._p(sequence_ids), ops._p(steps), int(step_offset), ops._stream()), "sample")
    return out


def history_window(histories: list[list[int]]) -> tuple[np.ndarray, np.ndarray]:
    """The last HISTORY_WINDOW tokens of each sequence as int32 [rows, 64] and their counts."""
    arr = np.full((len(histories), HISTORY_WINDOW), -1, dtype=np.int32)
    lens = np.zeros(len(histories), dtype=np.int32)
    for i, h in enumerate(histories):
        tail = h[-HISTORY_WINDOW:]
        arr[i, :len(tail)] = tail
        lens[i] = len(tail)
    return arr, lens
