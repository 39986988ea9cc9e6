"""One rank of the gathered column-sharded GEMM (run as a child process by test_peer_gather_gpu.py).

usage: peer_gather_worker.py RANK WORLD PORT M N_TOTAL K
Ranks use GPU ``rank % device_count``: with one GPU both ranks share it, which still exercises the export /
map / store-through-a-mapping path, because the mapping of another process's allocation is what the kernel
writes through either way. Rendezvous is gloo on 127.0.0.1; only the pickled handles travel through it.
Exits 0 when this rank's full matrix equals the CPU oracle's, bit for bit.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> int:
    rank, world, port, M, n_total, K = (int(v) for v in sys.argv[1:7])
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import qgemm_b200 as q
    from oracle import oracle as o
    from qgemm_b200 import datagen, sharding
    dev = torch.device("cuda", rank % torch.cuda.device_count())
    torch.cuda.set_device(dev)

    a_np = datagen.int8_uniform((M, K), seed=21, stream=0)        # replicated
    b_np = datagen.int8_uniform((n_total, K), seed=21, stream=1)  # every rank regenerates all of it
    n0, n1 = sharding.partition_columns(n_total, world, rank)
    a = torch.from_numpy(a_np).to(dev)
    b_slice = torch.from_numpy(np.ascontiguousarray(b_np[n0:n1])).to(dev)
    sa = torch.tensor([0.011], device=dev)
    sb = torch.tensor([0.017], device=dev)

    out = sharding.GatheredOutput(M, n_total, torch.bfloat16, dev)
    out.local.fill_(-5.0)
    torch.cuda.synchronize(dev)
    dist.barrier()  # nobody stores into a matrix that is still being filled
    for _ in range(2):  # a second pass over the same buffers must leave the same result
        sharding.sharded_mix_gemm_gather(a, b_slice, sa, sb, out)
    torch.cuda.synchronize(dev)
    dist.barrier()  # every rank's stores have landed
    rc, st = q.device_status()
    got = out.local.view(torch.int16).cpu().numpy().view(np.uint16)
    out.close()

    acc = o.gemm_i8(a_np, b_np, True)
    want = o.scale_cast(acc, 0.011, 0.017, o.OUT_BF16)
    # the device multiplies by fl(sa*sb) computed in float32 like the oracle; allow the documented 1 ulp
    ok = rc == 0 and o.bf16_ulp_distance(got, want) <= 1
    # and the blocks written by the other ranks are really theirs: compare with this rank's own kernel
    ref = torch.zeros((M, n_total), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, torch.from_numpy(b_np).to(dev), sa, sb, ref, b_kmajor=True)
    same = np.array_equal(got, ref.view(torch.int16).cpu().numpy().view(np.uint16))
    print(f"rank {rank}: status {rc} {st} oracle_ok {ok} equals_single_gpu {same}", flush=True)
    dist.destroy_process_group()
    return 0 if (ok and same) else 1


if __name__ == "__main__":
    sys.exit(main())
