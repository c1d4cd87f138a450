"""Host-side logic of the multi-GPU path, exercised with two gloo ranks on CPU."""
import os
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_images, q):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    sys.path.insert(0, str(root / 'kad-conv_b200'))
    import torch.distributed as dist
    from kadcnet.sharding import gather_detections, shard_range
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    a, b = shard_range(n_images, rank, world)
    # image i "detects" i % 3 boxes whose first coordinate is the image index
    local = [torch.full((i % 3, 6), float(i)) for i in range(a, b)]
    out = gather_detections(local, rank, world)
    if rank == 0:
        q.put([(t.shape[0], float(t[0, 0]) if t.shape[0] else -1.0) for t in out])
    else:
        assert out is None
    dist.barrier()
    dist.destroy_process_group()


def test_shard_ranges_cover_batch_once():
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / 'kad-conv_b200'))
    from kadcnet.sharding import shard_range
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_gather_on_gloo():
    world, n = 2, 7
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got == [(i % 3, float(i) if i % 3 else -1.0) for i in range(n)]
