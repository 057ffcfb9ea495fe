"""The N > 1 host logic (sequence sharding, barrier, max-over-ranks, aggregate rate) under
torch.distributed with the gloo backend, world size 2, on CPU."""
import os
import subprocess
import sys
import textwrap

import pytest

from homura_b200.replicas import aggregate_rate, shard_sequences

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shards_cover_every_sequence_once():
    for n, world in [(64, 8), (512, 8), (7, 2), (3, 4), (0, 2), (1, 1)]:
        seen = []
        for r in range(world):
            seen += list(shard_sequences(n, r, world))
        assert seen == list(range(n))
        sizes = [len(shard_sequences(n, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_sequences(4, 2, 2)
    assert aggregate_rate([128, 128], 0.5) == 512.0


WORKER = textwrap.dedent(
    """
    import sys
    sys.path.insert(0, %r)
    from homura_b200.replicas import Rendezvous, shard_sequences, aggregate_rate
    rv = Rendezvous("gloo")
    assert rv.world == 2
    mine = shard_sequences(9, rv.rank, rv.world)
    rv.barrier()
    t = rv.max(0.25 if rv.rank == 0 else 0.5)       # the slower rank sets the time
    units = rv.gather_ints(len(mine) * 10)
    rate = aggregate_rate(units, t)
    rv.barrier()
    if rv.rank == 0:
        print("RESULT", t, units, rate)
    rv.close()
    """
)


def test_two_ranks_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    port = 29500 + os.getpid() % 2000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT")][0]
    assert line == "RESULT 0.5 [50, 40] 180.0"
