"""The multi-rank host logic on CPU: world size 2 over gloo.  Each rank computes the attention of
its own batch slice with the CPU oracle (standing in for the GPU kernel, which needs no other rank),
the outputs are all-gathered, and the result must equal the unsharded computation."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _load_sharding():
    import importlib.util
    spec = importlib.util.spec_from_file_location("sfb_sharding", os.path.join(ROOT, "sf-bert_b200", "sharding.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, HERE)
    import torch.distributed as dist
    import oracle_lib as O
    sh = _load_sharding()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, L, H, d, bs = 4, 128, 2, 32, 32
    luts = O.lut_build(O.layout("local", 1, L // bs, left=1, right=1))
    q, k, v = (O.fill_normal((B, L, H, d), 70 + i) for i in range(3))
    b0, b1 = sh.batch_slice(B, world, rank)
    local = O.attention(q[b0:b1], k[b0:b1], v[b0:b1], luts, bs, np.float32(0.2), want=("o",))["o"]
    full = sh.gather_outputs(torch.from_numpy(local), world, dist)
    dist.barrier()
    if rank == 0:
        np.save(os.path.join(out_dir, "gathered.npy"), full.numpy())
    dist.destroy_process_group()


def test_partition_covers_every_pair_once():
    sh = _load_sharding()
    for batch, heads, world in [(8, 12, 8), (4, 16, 8), (3, 5, 4), (1, 4, 2), (2, 3, 7)]:
        seen = []
        for r in range(world):
            a, b = sh.partition_pairs(batch, heads, world, r)
            assert 0 <= a <= b <= batch * heads
            seen += list(range(a, b))
        assert seen == list(range(batch * heads))
    with pytest.raises(ValueError):
        sh.partition_pairs(2, 2, 2, 2)
    with pytest.raises(ValueError):
        sh.batch_slice(3, 2, 0)


def test_two_ranks_gather_equals_unsharded(tmp_path, oracle):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = np.load(tmp_path / "gathered.npy")
    B, L, H, d, bs = 4, 128, 2, 32, 32
    luts = oracle.lut_build(oracle.layout("local", 1, L // bs, left=1, right=1))
    q, k, v = (oracle.fill_normal((B, L, H, d), 70 + i) for i in range(3))
    want = oracle.attention(q, k, v, luts, bs, np.float32(0.2), want=("o",))["o"]
    assert np.array_equal(got, want)


def test_pair_slices_cover_a_rank_share_exactly():
    """bench.py turns a rank's contiguous range of (batch, head) pairs into rectangles of the [B, L, H, d] tensors (the head
    slices sfb_fused_attention_slice takes): every pair of the range exactly once, for every world size of the scaling run."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("sfb_bench", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    spec = importlib.util.spec_from_file_location("sfb_sharding", os.path.join(root, "sf-bert_b200", "sharding.py"))
    sh = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sh)
    for B, H in ((4, 16), (3, 5), (1, 7)):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for rank in range(world):
                start, stop = sh.partition_pairs(B, H, world, rank)
                for (b0, b1, h0, h1) in bench.pair_slices(B, H, start, stop):
                    assert 0 <= b0 < b1 <= B and 0 <= h0 < h1 <= H
                    seen += [b * H + h for b in range(b0, b1) for h in range(h0, h1)]
            assert sorted(seen) == list(range(B * H)) and len(seen) == B * H
