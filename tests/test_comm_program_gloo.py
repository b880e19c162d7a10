"""The op program ``CommGenerator.generate_code_for_plan`` emits, interpreted on two CPU ranks (gloo):
every rank walks its own ``CommInfo.operations`` - copy-engine copies as byte moves between the
ranks' buffer images, signal ops as writes to / checks of the ranks' flag arrays - and ends up with
the gathered buffer and with exactly the flags its lowered schedule waits for.  Host logic only:
no GPU, no CUDA call."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from syncopate_b200.operators import plan_all_gather

        dt = torch.bfloat16
        rows, K = 32, 16
        for split in (1, 2):
            _gen, info, low = plan_all_gather(world, rows, K, dt, "swizzle", copy_engine=True, chunk_split=split)
            g = torch.Generator().manual_seed(500 + rank)
            image = torch.zeros(world * rows, K, dtype=dt)
            image[rank * rows:(rank + 1) * rows] = torch.randn(rows, K, generator=g).to(dt)
            # every rank's buffer image before the program runs (a pull reads the owner's resident slab)
            images = [torch.empty_like(image) for _ in range(world)]
            dist.all_gather(images, image)
            mine = image.view(torch.uint8).reshape(-1).clone()
            flags = [0] * info.recv_signal_num
            for stream in info.operations[rank]:
                for op in stream:
                    kind = type(op).__name__
                    if kind == "CopyEngineOp":
                        assert op.dst_rank == rank and op.src == op.dst == "a"
                        src = images[op.src_rank].view(torch.uint8).reshape(-1)
                        mine[op.dst_offset:op.dst_offset + op.size] = src[op.src_offset:op.src_offset + op.size]
                    elif kind == "IntraNodeSignal":
                        assert op.rank == rank
                        flags[op.offset] = 1
                    else:
                        raise AssertionError(f"unexpected op {op}")
            gathered = mine.view(dt).reshape(world * rows, K)
            assert torch.equal(gathered, torch.cat([im[r * rows:(r + 1) * rows] for r, im in enumerate(images)], 0))
            sched = low[rank]["a"]
            waited = sorted(s for s in sched.gen_signal_lists() if s >= 0)
            assert waited == list(range(info.recv_signal_num)) and all(flags)
            # every wave's rows are exactly what one copy (or the resident slab) delivered
            assert sum(s[0] for s in sched.gen_block_shape_lists()) == world * rows
            assert len(sched.gen_signal_lists()) == 1 + (world - 1) * split
        results[rank] = "ok"
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_interpret_their_op_programs():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}
