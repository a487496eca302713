"""Host logic of the multi-GPU paths on CPU: shard boundaries, and (two gloo ranks) that
all-gathered column slabs reassemble the row-major tensor the single-device path produces."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import krea2_hrx_b200 as k
from krea2_hrx_b200 import parallel


def test_shard_columns_split_whole_tiles():
    assert parallel.shard_columns(15360, 2, 128) == [(0, 7680), (7680, 7680)]
    assert parallel.shard_columns(15360, 8, 128)[7] == (13440, 1920)
    assert parallel.shard_columns(32768, 8, 128)[3] == (12288, 4096)
    assert parallel.shard_columns(6144, 1, 128) == [(0, 6144)]
    with pytest.raises(k.InvalidArgument, match="do not split"):
        parallel.shard_columns(6144 + 128, 8, 128)
    with pytest.raises(k.InvalidArgument, match="world must be"):
        parallel.shard_columns(6144, 9, 128)
    # every share keeps gate|up pairs together: 32 interleaved rows = 16 outputs
    for first, count in parallel.shard_columns(32768, 8, 128):
        assert first % 32 == 0 and count % 32 == 0


def test_shard_rows_gives_equal_shares_and_a_short_last_one():
    assert parallel.shard_rows(4608, 8) == [(576 * r, 576) for r in range(8)]
    assert parallel.shard_rows(16896, 4)[3] == (12672, 4224)
    assert parallel.shard_rows(300, 4) == [(0, 75), (75, 75), (150, 75), (225, 75)]
    assert parallel.shard_rows(4115, 8)[7] == (3605, 510)  # 515 rows each, the last one shorter
    assert sum(count for _, count in parallel.shard_rows(4115, 8)) == 4115
    assert parallel.shard_rows(16, 1) == [(0, 16)]
    with pytest.raises(k.InvalidArgument, match="do not give each"):
        parallel.shard_rows(17, 8)  # shares of 3 rows leave the last two devices without one
    with pytest.raises(k.InvalidArgument, match="world must be"):
        parallel.shard_rows(64, 0)


def test_row_shares_cut_the_text_and_image_rows_without_gaps():
    """The token-sharded loop: each rank's rows of [text; image] as text rows plus a range of image rows; over the
    ranks the image ranges tile the image exactly, wherever the text/image boundary falls."""
    from krea2_hrx_b200 import pipeline
    for tokens, text_tokens, world in [(4608, 512, 8), (4608, 512, 4), (131, 70, 3), (300, 1, 4), (300, 299, 4), (16896, 512, 8)]:
        next_image, text_seen = 0, 0
        for first, count in parallel.shard_rows(tokens, world):
            text_count, image_first, image_count = pipeline.share_of_image(first, count, text_tokens)
            assert text_count + image_count == count and text_count >= 0 and image_count >= 0
            if image_count:
                assert image_first == next_image
                next_image += image_count
            text_seen += text_count
        assert next_image == tokens - text_tokens and text_seen == text_tokens
    assert pipeline.share_of_image(0, 44, 70) == (44, 0, 0)  # a rank of text rows only
    assert pipeline.share_of_image(44, 44, 70) == (26, 0, 18)
    assert pipeline.share_of_image(88, 43, 70) == (0, 18, 43)


def _row_gather_worker(rank, world, port, failures):
    """The token-sharded chain's NCCL baseline on gloo: equal padded shares all-gathered into the rows of the
    full K tensor; rows past the sequence land beyond `tokens` and are never read."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tokens, width = 37, 256
        gen = torch.Generator().manual_seed(9)
        want = torch.randn((tokens, width), generator=gen)
        first, count = parallel.shard_rows(tokens, world)[rank]
        share = -(-tokens // world)
        local = torch.zeros((share, width))
        local[:count] = want[first:first + count]
        full = torch.full((world * share + 3, width), 7.0)
        dist.all_gather_into_tensor(full[: world * share], local)
        if not torch.equal(full[:tokens], want):
            failures.put(f"rank {rank}: gathered rows differ")
        if not torch.equal(full[world * share:], torch.full((3, width), 7.0)):
            failures.put(f"rank {rank}: rows past the gathered range were written")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_gather_row_shares():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    procs = [ctx.Process(target=_row_gather_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert failures.empty(), failures.get()


def _gather_worker(rank, world, port, failures):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        rows, width = 37, 512
        want = torch.randn((rows, width), generator=gen)  # the same on every rank
        mine = torch.zeros_like(want)
        size = width // world
        mine[:, rank * size:(rank + 1) * size] = want[:, rank * size:(rank + 1) * size]  # this rank's slab only
        gathered = [torch.empty((rows, size)) for _ in range(world)]
        dist.all_gather(gathered, parallel.column_slab(mine, world, rank))
        parallel.assemble_columns(mine, torch.stack(gathered))
        if not torch.equal(mine, want):
            failures.put(f"rank {rank}: reassembled tensor differs")
        # data-parallel timing rule: the slowest rank defines the step
        t = torch.tensor([10.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if t.item() != 10.0 + world - 1:
            failures.put(f"rank {rank}: max-over-ranks gave {t.item()}")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reassemble_column_slabs():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert failures.empty(), failures.get()


def test_the_reference_arm_under_two_ranks_prints_one_line():
    """`bench.py --impl reference --gpus 2` under torchrun: rank 0 alone times the CPU port and prints the line,
    the other rank exits 0 without work."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(root, "bench.py"),
                           "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", "--cpu-tokens", "32"],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1 and lines[0]["impl"] == "reference" and lines[0]["n_gpus"] == 2
