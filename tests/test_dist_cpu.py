"""World-size-2 (and 3) gloo tests of the N-shard / gather logic on CPU.  The local GEMM is replaced by the
CPU oracle through the `compute` hook; the CUDA op itself never runs here."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_compute(xq, wq, sa, sw):
    from oracle import oracle as O

    return O.to_torch_bf16(O.c_matmul_blockwise(xq, wq, sa, sw))


def _worker(rank, world, port, N, fail_rank, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from gemm_int8_b200 import dist as gdist, workloads
        from oracle import oracle as O

        M, K = 24, 384
        x, y, sa, sw = workloads.nshard(M, N, K, seed=77)
        ys, sws = gdist.shard_weight(y, sw, rank, world)
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        full = gdist.matmul_blockwise_nsharded(x, ys, sa, sws, N, gather=True, row_major=True, compute=_oracle_compute)
        ref = O.c_matmul_blockwise(x, y, sa, sw)
        ok = np.array_equal(O.bf16_bits(full), ref)
        if gdist.uniform_shards(N, world):
            blocks = gdist.matmul_blockwise_nsharded(x, ys, sa, sws, N, gather=True, row_major=False,
                                                     compute=_oracle_compute)
            n = N // world
            ok = ok and all(np.array_equal(O.bf16_bits(blocks[r]), ref[:, r * n:(r + 1) * n]) for r in range(world))
        local = gdist.matmul_blockwise_nsharded(x, ys, sa, sws, N, gather=False, compute=_oracle_compute)
        n0, n1 = gdist.shard_bounds(N, world, rank)
        ok = ok and np.array_equal(O.bf16_bits(local), ref[:, n0:n1])
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"error: {type(e).__name__}: {e}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _kshard_worker(rank, world, port, N, fail_rank, q):
    """K-sharded (row-parallel) form: every rank holds a K slice; the ranks' fp32 partials are exchanged with one
    all-to-all and added in rank order.  The local GEMM and the ordered sum are the CPU oracle's."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from gemm_int8_b200 import dist as gdist, workloads
        from oracle import oracle as O

        M, K = 12 * world, 640   # five K blocks: ragged over 2 and 3 ranks
        x, y, sa, sw = workloads.nshard(M, N, K, seed=78)
        k0, k1 = gdist.kshard_bounds(K, world, rank)
        xs, ys = x[:, k0:k1].contiguous(), y[:, k0:k1].contiguous()
        sas, sws = sa[:, k0 // 128: -(-k1 // 128)].contiguous(), sw[:, k0 // 128: -(-k1 // 128)].contiguous()

        def compute(a, b, c, d):
            return torch.from_numpy(O.c_matmul_blockwise(a, b, c, d, return_acc=True)[1])

        def reduce(parts):
            tot = parts[0].numpy().copy()
            for r in range(1, parts.shape[0]):
                tot = (tot + parts[r].numpy()).astype(np.float32)
            return O.to_torch_bf16(O.np_bf16_rne(tot))

        rows = gdist.matmul_blockwise_ksharded(xs, ys, sas, sws, compute=compute, reduce=reduce)
        ref = O.c_matmul_blockwise_ksharded(x, y, sa, sw, world)
        m = M // world
        ok = rows.shape == (m, N) and np.array_equal(O.bf16_bits(rows), ref[rank * m:(rank + 1) * m])
        # and the sharded result stays within one bf16 ulp (plus the fp32 re-association floor) of the unsharded chain
        one = O.c_matmul_blockwise(x, y, sa, sw)[rank * m:(rank + 1) * m]
        ok = ok and int(O.bf16_ulp_distance(O.bf16_bits(rows), one).max()) <= 1
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"error: {type(e).__name__}: {e}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(world, N, fail_rank=-1, worker=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker or _worker, args=(r, world, port, N, fail_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


def test_shard_bounds_cover_and_align():
    from gemm_int8_b200 import dist as gdist

    for N in (128, 1000, 7168, 57344, 11008):
        for world in (1, 2, 3, 4, 8):
            prev = 0
            for r in range(world):
                n0, n1 = gdist.shard_bounds(N, world, r)
                assert n0 == prev and n0 % 128 == 0 and n1 >= n0
                prev = n1
            assert prev == N
    assert gdist.shard_bounds(57344, 8, 3) == (3 * 7168, 4 * 7168)
    assert gdist.uniform_shards(57344, 8) and not gdist.uniform_shards(11008, 4)
    with pytest.raises(ValueError):
        gdist.shard_bounds(128, 2, 2)


def test_assemble_row_major_layout():
    from gemm_int8_b200 import dist as gdist

    blocks = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = gdist.assemble_row_major(blocks)
    assert full.shape == (3, 8)
    assert torch.equal(full[:, :4], blocks[0]) and torch.equal(full[:, 4:], blocks[1])


def test_nshard_gather_world2_uniform():
    assert _run(2, 512) == {0: "ok", 1: "ok"}


def test_nshard_gather_world3_ragged():
    assert _run(3, 1000) == {0: "ok", 1: "ok", 2: "ok"}


def test_rank_failure_before_collective_is_reported_not_hung():
    """One rank raises before the gather: it reports its error; the survivor's collective ends with an error
    (process-group timeout / peer loss) instead of hanging."""
    res = _run(2, 512, fail_rank=1)
    assert res[1].startswith("error: RuntimeError: injected")
    assert res[0].startswith("error")


def test_kshard_reduce_scatter_world2_and_3():
    assert _run(2, 264, worker=_kshard_worker) == {0: "ok", 1: "ok"}
    assert _run(3, 136, worker=_kshard_worker) == {0: "ok", 1: "ok", 2: "ok"}
