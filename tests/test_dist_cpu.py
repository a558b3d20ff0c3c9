"""CPU tests of the multi-GPU plumbing (world_size 2, gloo): batch sharding, the weight-arena
broadcast and the id gather.  The data path itself has no collective."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from caten_b200 import dist as D
from caten_b200 import synthetic as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_batch_covers_the_batch_once():
    for batch in (1, 7, 64, 256):
        for world in (1, 2, 3, 4, 8):
            got = [D.shard_batch(batch, world, r) for r in range(world)]
            assert got[0][0] == 0
            for (b0, nb), (b1, _) in zip(got, got[1:]):
                assert b0 + nb == b1
            assert got[-1][0] + got[-1][1] == batch
            sizes = [nb for _, nb in got]
            assert max(sizes) - min(sizes) <= 1
    assert D.shard_batch(256, 8, 3) == (96, 32)
    with pytest.raises(ValueError):
        D.shard_batch(4, 2, 2)


def test_arena_roundtrip():
    p = S.GPT2Params(n_layers=1, n_heads=1, dim=64, vocab_size=97)
    sd = S.synth_state_dict(p, "q4_0", seed=2, max_seq_len=8, trivial_affine=False)
    arena, index = D.pack_arena(sd)
    assert all(e.offset % D.ALIGN == 0 for e in index.values())
    back = D.unpack_arena(arena, index)
    assert list(back) == list(sd)
    for k, v in sd.items():
        if isinstance(v, S.Packed):
            assert (back[k].ggml_type, back[k].rows, back[k].cols) == (v.ggml_type, v.rows, v.cols)
            np.testing.assert_array_equal(back[k].data, v.data)
        else:
            np.testing.assert_array_equal(back[k], v)


WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from caten_b200 import dist as D, synthetic as S
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    p = S.GPT2Params(n_layers=1, n_heads=1, dim=64, vocab_size=97)
    ref = S.synth_state_dict(p, "q8_0", seed=5, max_seq_len=8)
    arena, index = D.broadcast_state_dict(ref if rank == 0 else None, torch.device("cpu"))
    got = D.unpack_arena(arena.numpy(), index)
    for k, v in ref.items():
        a, b = (got[k].data, v.data) if isinstance(v, S.Packed) else (got[k], v)
        assert np.array_equal(a, b), k
    stubs, ptrs = D.device_views(arena, index)
    assert stubs["lm_head.weight"].rows == 97 and ptrs["wte.weight"] == arena.data_ptr() + index["wte.weight"].offset
    batch, steps = 5, 3
    b0, nb = D.shard_batch(batch, world, rank)
    local = torch.arange(steps * batch).reshape(steps, batch)[:, b0:b0 + nb].contiguous()
    allids = D.gather_ids(local, batch, world)
    assert torch.equal(allids, torch.arange(steps * batch).reshape(steps, batch)), allids
    dist.barrier()
    dist.destroy_process_group()
    sys.stdout.write("rank%d-ok " % rank)
    sys.stdout.flush()
""")


def test_broadcast_and_gather_world_size_2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("-ok") == 2, r.stdout


def test_c_abi_shard_agrees_with_host_shard():
    """`caten_b200_dist_shard` (what a Lisp host calls) cuts the batch exactly as `shard_batch`."""
    import ctypes as C

    from caten_b200 import _lib as L
    lib = L.load()
    for batch in (1, 7, 64, 256):
        for world in (1, 2, 3, 8):
            for r in range(world):
                first, count = C.c_int64(), C.c_int64()
                assert lib.caten_b200_dist_shard(batch, world, r, C.byref(first), C.byref(count)) == 0
                assert (first.value, count.value) == D.shard_batch(batch, world, r)
    assert lib.caten_b200_dist_shard(4, 2, 2, C.byref(first), C.byref(count)) == L.EINVAL
    # group calls without a context are refused before anything touches a GPU or NCCL
    assert lib.caten_b200_dist_init(None, 0, 2, None) == L.EINVAL
    assert lib.caten_b200_dist_gather_ids(None, None, 0, None) == L.EINVAL
    assert lib.caten_b200_dist_rank(None) == -1


def test_assemble_gathered_undoes_the_padding():
    batch, steps = 5, 3
    want = np.arange(steps * batch).reshape(steps, batch)
    for world in (1, 2, 3, 5):
        nb_max = max(D.shard_batch(batch, world, r)[1] for r in range(world))
        flat = np.full((world, steps * nb_max), -1, np.int64)
        for r in range(world):
            b0, nb = D.shard_batch(batch, world, r)
            blk = np.full((steps, nb_max), -1, np.int64)
            blk[:, :nb] = want[:, b0:b0 + nb]
            flat[r] = blk.reshape(-1)
        np.testing.assert_array_equal(D.assemble_gathered(flat, steps, batch, world), want)
