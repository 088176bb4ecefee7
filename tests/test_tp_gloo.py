"""N-sharded tensor-parallel wrapper on CPU ranks (gloo, world_size 2 and 4): sharding of
B / Bs, in-place all-gather layout and the final [M, N] assembly.  The per-rank matmul is
injected (the checker from oracle/), the code under test is the host-side plumbing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fp8_oracle as oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hf_kernels_helion_b200 import tp

        A, B, As, Bs = oracle.make_quantised_inputs(M, N, K, 0)   # every rank builds the same tensors from the seed
        calls = []

        def checker(a, b, sa, sb, block_size, dtype):
            calls.append((tuple(b.shape), tuple(sb.shape)))
            return oracle.w8a8_block_fp8_matmul(a, b, sa, sb, block_size, dtype)

        lin = tp.ShardedFp8Linear.from_full(B, Bs, matmul=checker)
        out = lin(A, As, torch.bfloat16)
        full = oracle.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
        slots = lin.forward_slots(A, As, torch.bfloat16)
        ok = (out.shape == (M, N) and out.is_contiguous() and torch.equal(out, full)
              and calls[0] == ((N // world, K), (N // world // 128, K // 128))
              and slots.shape == (world, M, N // world)
              and torch.equal(slots.permute(1, 0, 2).reshape(M, N), full)
              and lin.N == N)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_linear_matches_single_rank(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 48, 128 * world * 2, 256, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(world))
    assert results == {r: True for r in range(world)}
