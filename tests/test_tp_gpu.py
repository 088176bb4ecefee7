"""N-sharded tensor-parallel GEMM on real GPUs over NCCL (skipped with fewer than 2 GPUs)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fp8_oracle as oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hf_kernels_helion_b200 import runtime, tp

        M, N, K = 640, 256 * world, 1024
        A, B, As, Bs = oracle.make_quantised_inputs(M, N, K, 0)
        dev = torch.device("cuda", rank)
        lin = tp.ShardedFp8Linear.from_full(B.to(dev), Bs.to(dev))
        out = lin(A.to(dev), As.to(dev), torch.bfloat16)
        runtime.check_device_status()
        ref = oracle.gemm_dequant(A, B, As, Bs)
        ok = out.shape == (M, N) and oracle.bf16_ulp_error(out.cpu(), ref) <= 1
        # exchange fused into the GEMM epilogue (peer stores): same values, three calls to cycle the buffers
        for _ in range(3):
            fused = lin.forward_fused(A.to(dev), As.to(dev), torch.bfloat16)
            torch.cuda.synchronize()
            ok = ok and fused.shape == (M, N) and torch.equal(fused, out)
        runtime.check_device_status()
        # exchange through NVLink multicast (multimem.st, replicated by the NVSwitch), where the box has it;
        # fp32 output as well, whose rows are 4-byte elements in 128-byte boxes
        mc = torch.tensor([1.0 if tp.multicast_supported(dev) else 0.0], device=dev)
        dist.all_reduce(mc, op=dist.ReduceOp.MIN)
        used_mc = float(mc.item()) > 0
        if used_mc:
            for _ in range(3):
                got = lin.forward_multimem(A.to(dev), As.to(dev), torch.bfloat16)
                torch.cuda.synchronize()
                ok = ok and got.shape == (M, N) and torch.equal(got, out)
            got32 = lin.forward_multimem(A.to(dev), As.to(dev), torch.float32)
            torch.cuda.synchronize()
            ref32 = runtime.gemm(A.to(dev), B.to(dev), As.to(dev), Bs.to(dev), 128, 128, torch.float32)
            ok = ok and torch.equal(got32, ref32)
            runtime.check_device_status()
        q.put((rank, (bool(ok), used_mc)))
        # no rank may tear down its IPC / multicast mappings while a peer's kernels still use them
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_linear_nccl():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, val = q.get(timeout=300)
            res[rank] = val
        for p in procs:
            p.join(60)
    finally:
        # a worker that hangs (rendezvous, IPC open, a peer that died) must not outlive the test with
        # its GPU memory and kernels: end it by its own handle
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(5)
    assert [p.exitcode for p in procs] == [0] * world
    assert {r: v[0] for r, v in res.items()} == {r: True for r in range(world)}
    print("multimem exchange exercised:", all(v[1] for v in res.values()))
