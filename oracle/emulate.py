"""CPU oracle (TEST INFRASTRUCTURE, not product code): PyTorch-CPU emulation of the fused operators.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference arm may
import this module; the product never does.

What it restates.  The reference project defines the result of a fused operator as "run the
communication plan, then the plain operator" and checks its GPU kernels against exactly that:
``all_gather_into_tensor`` + ``matmul`` (tests/test_ag_gemm_gen.py:116-118), ``matmul`` +
``reduce_scatter_tensor`` (tests/test_gemm_rs.py:151-155), all-to-all + ``flash_attn_func``
(tests/test_all2all_attn_transform.py:157-200, :231-235), attention + all-to-all
(tests/test_attn_all2all_transform.py:88-103), KV all-gather + attention
(tests/test_allgather_attn_transform.py:148-168).  The functions below execute the LOWERED
schedule wave by wave (the order a fused kernel sees data arrive) on CPU tensors: a "transfer" is
a slice copy from the owner rank's tensor, "compute" is an fp32-accumulated matmul or an
fp32-softmax attention block with log-sum-exp merging (math of
syncopate/computation/attn/template.py:173-179, :222-231, :339-349, here in base e).

Pins.  (1) The schedule closed forms below are checked against the golden vectors generated from
the reference front end (tests/golden/frontend_golden.json).  (2) The chunk-ordered results are
checked to equal the un-chunked gather-then-operate results bit for bit (tests/test_oracle.py),
which is the reference's own definition of the golden output.  Causal masking, zigzag placement
and grouped-query attention have no counterpart in the reference (parity unpinned there); their
oracle is the dense fp32 computation in this file.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

# --------------------------------------------------------------------------- schedule closed forms


def swizzle_pull_schedule(world: int, rank: int, rows: int, cols: int) -> Dict[str, list]:
    """Lowered schedule of ``build_all_gather_plan_1d_swizzle(..., 'pull')`` for buffer rows:
    wave 0 is the resident slab, wave i the slab of rank (rank + i) % world with flag i - 1
    (syncopate/communication/common_descriptors/all_gather.py:77-96 + interface/lowering.py)."""
    order = [(rank + i) % world for i in range(world)]
    return {
        "offsets": [[p * rows, 0] for p in order],
        "shapes": [[rows, cols]] * world,
        "signals": [-1] + list(range(world - 1)),
        "targets": order,
    }


def ring_push_schedule(world: int, rank: int, rows: int, cols: int) -> Dict[str, list]:
    """Lowered schedule of ``build_ring_all_gather_plan``: slabs arrive from the upstream
    neighbour in the order rank, rank-1, rank-2, ... (all_gather.py:192-216)."""
    order = [(rank - i) % world for i in range(world)]
    up = (rank - 1) % world
    return {
        "offsets": [[p * rows, 0] for p in order],
        "shapes": [[rows, cols]] * world,
        "signals": [-1] + list(range(world - 1)),
        "targets": [rank] + [up] * (world - 1),
    }


def direct_reduce_schedule(world: int, rank: int, slab: int, cols: int) -> Dict[str, list]:
    """Lowered 'src' schedule of ``build_reduce_scatter_direct_reduce_plan(..., 'push')``: slabs
    of the partial result in the order rank+1, ..., rank-1, own last (reduce_scatter.py:238-302)."""
    order = [(rank + i + 1) % world for i in range(world)]
    return {
        "offsets": [[p * slab, 0] for p in order],
        "shapes": [[slab, cols]] * world,
        "signals": list(range(world)),
        "targets": order[:-1] + [-1],
    }


# --------------------------------------------------------------------------- GEMM operators


def gather_by_schedule(schedule: Dict[str, list], shards: Sequence[torch.Tensor]) -> torch.Tensor:
    """Executes the waves of a gathered-buffer schedule: every block is copied from its owner."""
    rows = shards[0].shape[0]
    out = torch.empty(rows * len(shards), shards[0].shape[1], dtype=shards[0].dtype)
    for off, shp in zip(schedule["offsets"], schedule["shapes"]):
        owner, inner = divmod(off[0], rows)
        out[off[0] : off[0] + shp[0], off[1] : off[1] + shp[1]] = shards[owner][
            inner : inner + shp[0], off[1] : off[1] + shp[1]
        ]
    return out


def ag_gemm(schedule: Dict[str, list], shards: Sequence[torch.Tensor], b: torch.Tensor,
            out_dtype: Optional[torch.dtype] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather + GEMM in arrival order.  ``shards[r]`` is rank r's ``[rows, K]`` slab, ``b`` is
    ``[N, K]``.  Returns (gathered A, C = A @ b^T) with fp32 accumulation, C cast to ``out_dtype``."""
    rows, K = shards[0].shape
    M = rows * len(shards)
    gathered = torch.empty(M, K, dtype=shards[0].dtype)
    c = torch.empty(M, b.shape[0], dtype=torch.float32)
    bt = b.to(torch.float32).t().contiguous()
    for off, shp in zip(schedule["offsets"], schedule["shapes"]):
        owner, inner = divmod(off[0], rows)
        block = shards[owner][inner : inner + shp[0]]
        gathered[off[0] : off[0] + shp[0]] = block
        c[off[0] : off[0] + shp[0]] = block.to(torch.float32) @ bt
    return gathered, c.to(out_dtype or shards[0].dtype)


def gemm_rs(schedules: Sequence[Dict[str, list]], a: Sequence[torch.Tensor], b: Sequence[torch.Tensor],
            out_dtype: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """GEMM + reduce-scatter.  ``a[r]`` ``[M, K_r]``, ``b[r]`` ``[N, K_r]``; rank r walks its
    partial-product schedule ``schedules[r]`` slab by slab, each slab is added (fp32) into its
    owner's output.  Returns the per-rank ``[M / world, N]`` outputs."""
    world = len(a)
    M, N = a[0].shape[0], b[0].shape[0]
    slab = M // world
    acc = [torch.zeros(slab, N, dtype=torch.float32) for _ in range(world)]
    for r in range(world):
        bt = b[r].to(torch.float32).t().contiguous()
        for off, shp in zip(schedules[r]["offsets"], schedules[r]["shapes"]):
            owner, inner = divmod(off[0], slab)
            part = a[r][off[0] : off[0] + shp[0]].to(torch.float32) @ bt
            acc[owner][inner : inner + shp[0]] += part
    dt = out_dtype or a[0].dtype
    return [x.to(dt) for x in acc]


# --------------------------------------------------------------------------- attention


def attention_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float,
                    q_pos: Optional[torch.Tensor] = None, k_pos: Optional[torch.Tensor] = None,
                    causal: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax attention for ``q [Hq, Sq, D]``, ``k, v [Hkv, Sk, D]`` (Hq a multiple of Hkv:
    grouped-query heads share a KV head).  ``causal`` masks key j for query i unless
    ``k_pos[j] <= q_pos[i]`` (true token positions).  Returns (out fp32, lse natural-log)."""
    hq, sq, d = q.shape
    hkv = k.shape[0]
    group = hq // hkv
    qf, kf, vf = q.float(), k.float(), v.float()
    out = torch.empty(hq, sq, d, dtype=torch.float32)
    lse = torch.empty(hq, sq, dtype=torch.float32)
    mask = None
    if causal:
        qp = torch.arange(sq) if q_pos is None else q_pos
        kp = torch.arange(k.shape[1]) if k_pos is None else k_pos
        mask = kp[None, :] > qp[:, None]
    for h in range(hq):
        s = (qf[h] @ kf[h // group].t()) * sm_scale
        if mask is not None:
            s = s.masked_fill(mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        out[h] = (p @ vf[h // group]) / torch.where(l == 0, torch.ones_like(l), l)
        lse[h] = (m + torch.log(l)).squeeze(-1)
    return out, lse


def merge_partials(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor):
    """Log-sum-exp merge of two normalised partial attention results over disjoint key sets
    (syncopate/computation/attn/template.py:339-349, base e here)."""
    m = torch.maximum(lse1, lse2)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m_safe), torch.exp(lse2 - m_safe)
    tot = w1 + w2
    tot_safe = torch.where(tot == 0, torch.ones_like(tot), tot)
    o = (o1 * w1[..., None] + o2 * w2[..., None]) / tot_safe[..., None]
    return o, m_safe + torch.log(tot)


def attention_by_blocks(q, k, v, sm_scale, blocks, q_pos=None, k_pos=None, causal=False):
    """Attention executed as an ordered list of ``(q_lo, q_len, kv_lo, kv_len)`` blocks (the
    (Q, KV) axes of a lowered attention schedule), merging partial results per query row."""
    hq, sq, d = q.shape
    out = torch.zeros(hq, sq, d, dtype=torch.float32)
    lse = torch.full((hq, sq), float("-inf"))
    qp = torch.arange(sq) if q_pos is None else q_pos
    kp = torch.arange(k.shape[1]) if k_pos is None else k_pos
    for q_lo, q_len, kv_lo, kv_len in blocks:
        qs, ks = slice(q_lo, q_lo + q_len), slice(kv_lo, kv_lo + kv_len)
        o_b, l_b = attention_dense(q[:, qs], k[:, ks], v[:, ks], sm_scale, qp[qs], kp[ks], causal)
        o_m, l_m = merge_partials(out[:, qs], lse[:, qs], o_b, l_b)
        out[:, qs], lse[:, qs] = o_m, l_m
    return out, lse


def zigzag_positions(world: int, rank: int, chunk: int) -> torch.Tensor:
    """True token positions of rank ``rank``'s queries under zigzag context parallelism: chunks
    ``rank`` and ``2 * world - 1 - rank`` of ``2 * world`` equal chunks."""
    a = torch.arange(rank * chunk, (rank + 1) * chunk)
    b = torch.arange((2 * world - 1 - rank) * chunk, (2 * world - rank) * chunk)
    return torch.cat([a, b])
