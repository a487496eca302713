"""One rank of the column-sharded chain (launched by torchrun, one process per GPU).

--check: small dimensions, fused push and NCCL baseline both compared bit for bit with the
         single-device session run on this rank's GPU.
--time:  the reference's dimensions over a few layers; prints the per-forward device time of the
         single-device session, the fused push and the NCCL baseline (max over ranks).
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import session_oracle as so  # noqa: E402


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--check", action="store_true")
    parser.add_argument("--time", action="store_true")
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--tokens", type=int, default=4608)
    parser.add_argument("--iters", type=int, default=5)
    args = parser.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import krea2_hrx_b200 as k
    from krea2_hrx_b200 import parallel, session
    stream = torch.cuda.current_stream()
    if args.check:
        dims, layers, tokens = session.ModelDims(**so.SMALL), 2, 300
    else:
        dims, layers, tokens = session.ModelDims(), args.layers, args.tokens
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(11, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=3)
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    mods_dev = torch.from_numpy(mods).cuda()
    single = session.Session(stream, weights, tokens, layers)
    single.set_attention(False)  # the sharded chain is the W8A8 chain
    fabric = parallel.SymmetricFabric()
    tp = parallel.TensorParallel(fabric, rank, dims, parallel.shard_weights(weights, layers, world, rank), tokens)
    fabric.barrier()

    def bits(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    if args.check:
        want = x_dev.clone()
        single.run_device(stream, want, mods_dev, torch.from_numpy(cos), torch.from_numpy(sin))
        torch.cuda.synchronize()
        for collective in ("fused", "nccl", "fused", "graph", "graph"):
            out = tp.forward_graph(x_dev, mods_dev) if collective == "graph" else tp.forward(x_dev, mods_dev, collective)
            fabric.barrier()
            if not np.array_equal(bits(out), bits(want)):
                print(f"rank {rank}: {collective} result differs", flush=True)
                sys.exit(1)
        if k.device_status() != 0:
            print(f"rank {rank}: device status raised", flush=True)
            sys.exit(1)
        fabric.barrier()
        if rank == 0:
            print("tp check ok", flush=True)
    if args.time:
        def timed(fn):
            for _ in range(2):
                fn()
            fabric.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(args.iters):
                fn()
            end.record(stream)
            fabric.barrier()
            t = torch.tensor([start.elapsed_time(end) / args.iters], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
        base = timed(lambda: single.run_device(stream, x_dev.clone(), mods_dev, torch.from_numpy(cos), torch.from_numpy(sin)))
        fused = timed(lambda: tp.forward(x_dev, mods_dev, "fused"))
        nccl = timed(lambda: tp.forward(x_dev, mods_dev, "nccl"))
        graph = timed(lambda: tp.forward_graph(x_dev, mods_dev))
        if rank == 0:
            print({"world": world, "layers": layers, "tokens": tokens, "single_gpu_ms": base, "tp_fused_eager_ms": fused,
                   "tp_nccl_eager_ms": nccl, "tp_fused_graph_ms": graph}, flush=True)
    single.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
