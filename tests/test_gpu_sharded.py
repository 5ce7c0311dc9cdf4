"""The sharded operator on real GPUs (needs at least two B200s; skipped otherwise).

One process per GPU over NCCL, NVLS disabled (no multicast objects are involved in this path).
Covers both shard plans: whole heads per rank (no collective) and the rows of one head split
zig-zag over the ranks with one all-reduce of the fp32 column vectors.
"""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, bh, m, n, causal, reduction, out_dir):
    import torch.distributed as dist

    from conftest import assert_parity
    from flash_colreduce_b200.sharding import NativeComm, plan_shards, sharded_colreduce, sharded_colreduce_native
    from oracle import oracle_colreduce

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["FCR_DEBUG_SYNC"] = "1"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(3)
        q = torch.randn(1, bh, m, 64, generator=g).half()
        k = torch.randn(1, bh, n, 64, generator=g).half()
        spec = plan_shards(bh, m, world, rank)
        out = sharded_colreduce(q[:, spec.head_lo:spec.head_hi].to(dev), k[:, spec.head_lo:spec.head_hi].to(dev),
                                reduction, causal, spec=spec, total_heads=bh)
        want = oracle_colreduce(q, k, reduction, causal)[0]
        assert out.shape == want.shape and out.dtype == torch.float16
        assert_parity(out, want, reduction, extra_rtol=2.0 ** -11)
        # the same through the library's own entry point: shard plan, kernels, ncclAllReduce and the
        # mean / cast queued by one C call on a communicator the library made
        comm = NativeComm()
        try:
            for _ in range(2):
                native = sharded_colreduce_native(q[:, spec.head_lo:spec.head_hi].to(dev), k[:, spec.head_lo:spec.head_hi].to(dev),
                                                  reduction, causal, total_heads=bh, comm=comm, world=world, rank=rank)
            torch.cuda.synchronize()
            assert native.shape == want.shape and native.dtype == torch.float16
            assert_parity(native, want, reduction, extra_rtol=2.0 ** -11)
            if reduction == "max":
                assert torch.equal(native, out)  # max does not depend on the order of combination
        finally:
            comm.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bh,m,n,causal,reduction", [
    (4, 700, 900, True, "mean"),    # heads partitioned
    (1, 3000, 3000, True, "sum"),   # rows of one head split zig-zag over the ranks
    (1, 1500, 520, True, "max"),    # M > N
    (1, 1024, 2048, False, "mean"),
    (3, 2000, 2000, True, "sum"),   # fewer heads than ranks on four GPUs: idle rank, one rank per head
])
def test_sharded_on_gpus(tmp_path, bh, m, n, causal, reduction):
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_worker, args=(world, _free_port(), bh, m, n, causal, reduction, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]
