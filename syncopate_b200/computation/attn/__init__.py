"""Host-side entry point of the attention kernel, with the argument conventions of the reference's
generated ``attention_forward`` (syncopate/computation/transform/transformer.py:1125-1178, used as in
tests/test_all2all_attn_transform.py:286-294): wave metadata over the axes (Z, H, Q, KV) in tokens,
a signal array with one flag index per wave, and an optional output buffer.

Additions of this backend: ``causal`` with true-position tables (``q_pos`` / ``kv_pos`` per 128 rows /
keys), grouped-query heads (``k`` / ``v`` may have fewer heads than ``q``), and an ``AttentionState``
that keeps the LSE / visit scratch between calls.  The work-balanced ownership plans
(``syn_attention_plan``) of the configurations seen so far are kept in a small module-level cache.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import torch

from syncopate_b200 import _lib as L

_DTYPES = {torch.float16: L.SYN_DTYPE_F16, torch.bfloat16: L.SYN_DTYPE_BF16}


class AttentionState:
    """Per-output scratch of the attention kernel: log2-domain LSE and the visit epochs that tell a
    first visit of a query row from a merge.  One state per output tensor; reuse it across calls."""

    def __init__(self, Z: int, H: int, Sq: int, device):
        self.lse = torch.empty(Z, H, Sq, dtype=torch.float32, device=device)
        self.visit = torch.zeros(Z, H, Sq, dtype=torch.int32, device=device)
        self.epoch = 0

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


def _strides3(t: torch.Tensor):
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("attention tensors must be [Z, H, S, D] views with a contiguous head dimension")
    return (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _tolist(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().tolist()
    return x


_PLAN_MAX_PAIRS_PER_CTA = 8
_PLANS: dict = {}  # configuration key -> AttnPlan, or None where the library declined to plan
_PLANS_MAX = 256


def _owner_plan(a: L.AttnArgs, sched, key, q_pos, kv_pos):
    """The ownership plan for this configuration, made on first use (host work, one device-to-host
    copy of the position tables) and kept."""
    if key not in _PLANS:
        if len(_PLANS) >= _PLANS_MAX:
            _PLANS.pop(next(iter(_PLANS)))
        qh = q_pos.detach().to("cpu", torch.int32).contiguous() if q_pos is not None else None
        kh = kv_pos.detach().to("cpu", torch.int32).contiguous() if kv_pos is not None else None
        plan = L.AttnPlan()
        rc = L.lib().syn_attention_plan(C.byref(a), C.byref(sched), qh.data_ptr() if qh is not None else None,
                                        kh.data_ptr() if kh is not None else None, C.byref(plan))
        if rc == L.SYN_ERR_TOO_LARGE:
            plan = None  # more units than a plan holds: arithmetic ownership
        else:
            L.check(rc, "syn_attention_plan")
        _PLANS[key] = plan
    return _PLANS[key]


def attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    output_buffer: Optional[torch.Tensor] = None,
    *,
    wave_offsets=None,
    wave_sizes=None,
    cum_wave_sizes=None,
    signal_ptr=None,
    signal_offsets=None,
    counter_ptr=None,
    NUM_WAVES: Optional[int] = None,
    cum_tiles: Optional[int] = None,
    causal: bool = False,
    q_pos: Optional[torch.Tensor] = None,
    kv_pos: Optional[torch.Tensor] = None,
    state: Optional[AttentionState] = None,
    signal_value: int = 1,
    comm: Optional[L.AttnComm] = None,
    push: Optional[L.AttnPush] = None,
    num_sms: int = 0,
    timeout_ns: int = 0,
    status=None,
    stream=None,
    balance: bool = True,
) -> torch.Tensor:
    """``softmax(q k^T * sm_scale) v`` over the given waves.  ``q`` ``[Z, Hq, Sq, 128]``, ``k`` / ``v``
    ``[Z, Hkv, Skv, 128]`` (any strides with the head dimension contiguous).  Without wave
    metadata one wave covers everything.  ``cum_wave_sizes``, ``NUM_WAVES``, ``cum_tiles`` and
    ``counter_ptr`` are accepted for signature compatibility (they follow from the waves).
    ``balance`` plans a work-balanced ownership of the query tiles on the first call of a
    configuration and reuses it afterwards.  ``push`` switches the kernel's producer role on (see
    ``syn_attn_push``): rows leave for their destination ranks at their tile's last visit instead of
    being stored to the output; it needs the planned ownership.
    Returns the output (``output_buffer`` if given)."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda or t.dtype not in _DTYPES:
            raise ValueError(f"{name} must be a CUDA fp16/bf16 tensor")
    Z, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    out = output_buffer if output_buffer is not None else torch.empty_like(q)
    if state is None:
        state = AttentionState(Z, Hq, Sq, q.device)
    a = L.AttnArgs()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse, a.visit = state.lse.data_ptr(), state.visit.data_ptr()
    a.Z, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = Z, Hq, Hkv, Sq, Skv, D
    a.q_strides, a.k_strides, a.v_strides, a.o_strides = _strides3(q), _strides3(k), _strides3(v), _strides3(out)
    a.sm_scale = float(sm_scale)
    a.causal = 1 if causal else 0
    a.q_pos = q_pos.data_ptr() if q_pos is not None else None
    a.kv_pos = kv_pos.data_ptr() if kv_pos is not None else None
    a.dtype = _DTYPES[q.dtype]
    a.num_sms = num_sms
    a.epoch = state.next_epoch()
    a.signal_ptr = signal_ptr.data_ptr() if isinstance(signal_ptr, torch.Tensor) else signal_ptr
    a.signal_value = signal_value
    a.timeout_ns = timeout_ns
    a.status = status.data_ptr() if isinstance(status, torch.Tensor) else status
    offs, sizes = _tolist(wave_offsets), _tolist(wave_sizes)
    if offs is None:
        offs, sizes = [[0, 0, 0, 0]], [[Z, Hq, Sq, Skv]]
    sched, keep = L.make_schedule(offs, sizes, _tolist(signal_offsets), ndim=4)
    if push is not None:
        if not balance:
            raise ValueError("the producer role needs the planned ownership (balance=True)")
        a.push = C.addressof(push)
    if balance and push is None:
        # Planned ownership pays when a CTA holds only a few tile pairs of different length (cfg3 per
        # rank: 3.5 per CTA, 1.01 ms planned against 1.13 ms arithmetic); with many pairs per CTA the
        # arithmetic rule balances as well and keeps neighbouring CTAs on the same heads (cfg4 per rank:
        # 13.8 per CTA, 8.8 ms arithmetic against 9.5 ms planned).
        sms = num_sms or torch.cuda.get_device_properties(q.device).multi_processor_count
        if Z * Hq * ((Sq + 255) // 256) > _PLAN_MAX_PAIRS_PER_CTA * sms:
            balance = False
    if balance:
        key = (os.environ.get("SYNCOPATE_B200_ATTN_TWO_TILE"), push is not None, Z, Hq, Hkv, Sq, Skv, bool(causal), num_sms, tuple(map(tuple, offs)), tuple(map(tuple, sizes)),
               None if q_pos is None else (q_pos.data_ptr(), q_pos._version),
               None if kv_pos is None else (kv_pos.data_ptr(), kv_pos._version))
        plan = _owner_plan(a, sched, key, q_pos, kv_pos)
        a.plan = C.addressof(plan) if plan is not None else None
        if push is not None and plan is None:
            raise L.SynError(L.SYN_ERR_TOO_LARGE, "attention_forward", "too many units for the producer role's plan")
    if stream is None:
        stream = torch.cuda.current_stream()
    rc = L.lib().syn_attention(C.byref(a), C.byref(sched), C.byref(comm) if comm is not None else None,
                               stream.cuda_stream or None)
    L.check(rc, "syn_attention")
    return out


__all__ = ["attention_forward", "AttentionState"]
