"""One rank of the sharded chains (launched by torchrun, one process per GPU), small dimensions.

Column-sharded weights (fused push, NCCL baseline, eager and graph replay) and token-sharded rows are each
compared bit for bit with the single-device session run on this rank's GPU.  The verdict is collective: after
every forward the ranks agree (an all-reduce of a per-rank flag) on whether all of them matched, so that on a
mismatch every rank synchronises, leaves the process group and exits non-zero TOGETHER -- no rank walks away
while a peer's kernels may still be storing into its buffers.  NVLS is switched off for the run (the launcher
sets NCCL_NVLS_ENABLE=0): no buffer is bound to an NVLink multicast object.
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
    parser.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import krea2_hrx_b200 as k
    from krea2_hrx_b200 import parallel, session
    stream = torch.cuda.current_stream()
    dims, layers, tokens = session.ModelDims(**so.SMALL), 2, 64 * world + 32
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(11, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=3)
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    mods_dev = torch.from_numpy(mods).cuda()
    cos_t, sin_t = torch.from_numpy(cos), torch.from_numpy(sin)
    single = session.Session(stream, weights, tokens, layers)
    fabric = parallel.SymmetricFabric()

    def bits(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    def agreed(ok: bool) -> bool:
        """True when every rank's forward matched; every rank learns the same answer."""
        torch.cuda.synchronize()
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item())

    held = {}  # the sharded runners: dropped (with their recorded graphs) before the process group goes

    def say(text: str):
        if rank == 0:
            print(text, flush=True)

    def leave(code: int):
        import gc
        torch.cuda.synchronize()
        fabric.barrier()
        held.clear()
        gc.collect()
        torch.cuda.empty_cache()
        single.close()
        fabric.barrier()
        dist.destroy_process_group()
        sys.exit(code)

    # column-sharded weights: the W8A8 chain
    single.set_attention(False)
    want = x_dev.clone()
    single.run_device(stream, want, mods_dev, cos_t, sin_t)
    torch.cuda.synchronize()
    tp = held["tp"] = parallel.TensorParallel(fabric, rank, dims, parallel.shard_weights(weights, layers, world, rank), tokens)
    fabric.barrier()
    for mode in ("fused", "nccl", "fused", "graph fused", "graph fused", "graph nccl", "graph nccl"):
        if mode.startswith("graph"):
            out = tp.forward_graph(x_dev, mods_dev, mode.split()[1])
        else:
            out = tp.forward(x_dev, mods_dev, mode)
        fabric.barrier()
        if not agreed(np.array_equal(bits(out), bits(want))):
            say(f"column-sharded chain ({mode}): a rank's result differs")
            leave(1)
        say(f"column-sharded chain ({mode}): ok")
    del tp
    held.clear()
    # token-sharded rows: the full block, attention on
    single.set_attention(True)
    want = x_dev.clone()
    single.run_device(stream, want, mods_dev, cos_t, sin_t)
    torch.cuda.synchronize()
    sp = held["sp"] = parallel.TokenParallel(fabric, rank, weights, tokens, layers)
    fabric.barrier()
    for mode in ("push", "nccl", "graph push", "graph push", "graph nccl"):
        graph, collective = mode.startswith("graph"), mode.split()[-1]
        out = sp.forward(x_dev, mods_dev, cos_t, sin_t, collective=collective, graph=graph)
        fabric.barrier()
        first, count = sp.rows
        if not agreed(np.array_equal(bits(out), bits(want[first:first + count]))):
            say(f"token-sharded chain ({mode}): a rank's rows differ")
            leave(1)
        say(f"token-sharded chain ({mode}): ok")
    del sp
    if not agreed(k.device_status() == 0):
        say("a rank's device status was raised")
        leave(1)
    say("tp check ok")
    leave(0)


if __name__ == "__main__":
    main()
