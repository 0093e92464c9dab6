"""One gloo rank of the CPU tensor-parallel test: python tp_rank_worker.py RANK WORLD PORT MODE OUT.npy"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(HERE), HERE]


def main() -> None:
    rank, world, port, mode, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    import torch
    import torch.distributed as dist

    import oracle
    from helpers import synth_weights
    from ojas_engine_b200 import Q4_K, tp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    if mode.startswith("absent-"):
        # failure detection on the host: rank 1 joins the group and then leaves between steps without taking part in the
        # collective; rank 0's join must end with an error after the group's timeout instead of hanging
        import datetime
        mode = mode[len("absent-"):]
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        if rank == 1:
            with open(out, "w") as fh:
                fh.write("left")
            os._exit(0)
        n, k, m = 50, 768, 2
        raw = synth_weights(Q4_K, n, k)
        x = np.random.default_rng(1).standard_normal((m, k)).astype(np.float32)
        sh = tp.ShardedLinear(raw, Q4_K, n, k, mode, rank, world)
        rows, klen = sh.local_shape
        y_local = torch.from_numpy(oracle.matmul_kq(sh.raw, Q4_K, rows, klen, sh.local_x(x), threads=1))
        try:
            sh.join(y_local, dist)
            verdict = "joined"
        except Exception as exc:           # the collective reports the missing rank
            verdict = "error: " + type(exc).__name__
        with open(out, "w") as fh:
            fh.write(verdict)
        os._exit(0)                         # the group is broken: no orderly shutdown
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, k, m = 50, 768, 2      # 50 rows over 2 ranks: equal shards; 768 = 3 super-blocks: uneven K shards
        raw = synth_weights(Q4_K, n, k)
        x = np.random.default_rng(1).standard_normal((m, k)).astype(np.float32)
        sh = tp.ShardedLinear(raw, Q4_K, n, k, mode, rank, world)
        rows, klen = sh.local_shape
        y_local = torch.from_numpy(oracle.matmul_kq(sh.raw, Q4_K, rows, klen, sh.local_x(x), threads=1))
        y = sh.join(y_local, dist)
        np.save(out, y.numpy())
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
