"""One rank of the multi-GPU tensor-parallel test (one process per GPU):
    python tp_gpu_worker.py RANK WORLD PORT
Llama-70B-shaped projections sharded over the ranks.  M = 1: the GEMV's peer-store epilogue + the bounded-wait join
(column-parallel QKV, gate/up; row-parallel O, down).  M = 512: the tensor-core GEMM + NCCL all-gather / all-reduce.
Every rank checks the JOINED result against the CPU oracle and exits non-zero on a mismatch."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.dirname(HERE), HERE]

TOL = 2e-3


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def main() -> None:
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    small = len(sys.argv) > 4 and sys.argv[4] == "small"
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    import oracle
    import ojas_engine_b200 as ob
    from ojas_engine_b200 import Q4_K, Q6_K, tp

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    gpu = ob.B200Gpu(rank)
    failures = []
    try:
        def exchange(blob):
            out = [None] * world
            dist.all_gather_object(out, blob)
            return out

        projections = [("qkv", Q4_K, 10240, 8192, "col"), ("o", Q4_K, 8192, 8192, "row"),
                       ("gate_up", Q4_K, 28672, 8192, "col"), ("down", Q6_K, 8192, 28672, "row")]
        if small:
            projections = [("qkv", Q4_K, 1280, 2048, "col"), ("down", Q6_K, 1024, 3584, "row")]
        group = tp.TpGroup(gpu, world, rank, max(p[2] for p in projections), exchange)
        stream = torch.cuda.ExternalStream(gpu.stream, device=f"cuda:{rank}")
        rng = np.random.default_rng(123)                      # the same inputs on every rank
        for name, t, n, k, mode in projections:
            raw = oracle.synth_blocks(t, n * k // 256)
            sh = tp.ShardedLinear(raw, t, n, k, mode, rank, world)
            rows, klen = sh.local_shape
            w = gpu.load_weight(sh.raw, t, rows, klen)
            # ---- M = 1: peer-store epilogue + join, three steps in a row (both halves of the windows, and a replayed graph)
            x = (rng.standard_normal((1, k)) * 0.1).astype(np.float32)
            want = oracle.matvec_kq(raw, t, n, k, x[0])
            xb = gpu.upload(sh.local_x(x))
            y = gpu.alloc(n)
            for step in range(3):
                gpu.memset(y, 0)
                group.gemv(w, xb)
                group.join(group.COL if mode == "col" else group.ROW, y, n)
                got = gpu.read(y, np.float32, n)
                err = rel_l2(got, want)
                if err > 1e-5:
                    failures.append(f"{name} M=1 step {step}: rel L2 {err:.3e}")
            gpu.graph_begin()
            group.gemv(w, xb)
            group.join(group.COL if mode == "col" else group.ROW, y, n)
            g = gpu.graph_end()
            for _ in range(3):                                 # an odd number of replays: the halves alternate on the device
                gpu.memset(y, 0)
                gpu.graph_launch(g)
                got = gpu.read(y, np.float32, n)
                if rel_l2(got, want) > 1e-5:
                    failures.append(f"{name} M=1 graph replay: rel L2 {rel_l2(got, want):.3e}")
            gpu.graph_destroy(g)
            # ---- M = 512: tensor-core GEMM + NCCL collective; sampled tokens against the oracle
            m = 64 if small else 512
            xm = (rng.standard_normal((m, k)) * 0.1).astype(np.float32)
            xmb = gpu.upload(sh.local_x(xm))
            yl = torch.empty(m, rows, device=f"cuda:{rank}", dtype=torch.float32)
            gpu.gemm(w, xmb, ob.Buf(yl.data_ptr(), yl.numel() * 4), m)
            gpu.sync()
            with torch.cuda.stream(stream):
                full = sh.join(yl, dist)
            torch.cuda.synchronize()
            sample = [0, m // 3, m - 1]
            wantm = oracle.matmul_kq(raw, t, n, k, xm[sample])
            errm = rel_l2(full[sample].cpu().numpy(), wantm)
            if errm > TOL:
                failures.append(f"{name} M={m}: rel L2 {errm:.3e}")
            for b in (w.buf, xb, y, xmb):
                gpu.free(b)
        # the one-kernel all-gather: every rank contributes a vector that names it
        nfl = 4096
        src = gpu.upload(np.full(nfl, float(rank + 1), np.float32) + np.arange(nfl, dtype=np.float32) / 8192)
        y_all = gpu.alloc(world * nfl)
        for _ in range(3):
            gpu.memset(y_all, 0)
            group.allgather(src, nfl, y_all)
            got = gpu.read(y_all, np.float32, world * nfl).reshape(world, nfl)
            want = np.stack([np.full(nfl, float(r + 1), np.float32) + np.arange(nfl, dtype=np.float32) / 8192 for r in range(world)])
            if not np.array_equal(got, want):
                failures.append("allgather mismatch")
        dist.barrier()
        group.close()
    finally:
        dist.destroy_process_group()
        gpu.close()
    if failures:
        print(f"rank {rank} FAILED: " + "; ".join(failures), flush=True)
        sys.exit(1)
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
