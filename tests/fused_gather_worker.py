"""Worker for the fused GEMM + all-gather check: run under torchrun (one process per GPU of one box).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/fused_gather_worker.py [--time]

Every rank computes its column shard with the gathering kernel, which writes into all ranks' full matrices; after the
barrier every rank compares ITS full matrix with the single-GPU kernel's result on the unsharded weight (bit-exact).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    import gemm_int8_b200 as g
    from gemm_int8_b200 import dist as gdist

    timed = "--time" in sys.argv
    shapes = [(300, 1024, 640), (1024, 4096, 2048)] + ([(16384, 57344, 8192)] if timed else [])
    ok = True
    for (M, N, K) in shapes:
        gen = torch.Generator().manual_seed(1234)  # the same operands on every rank
        if M * K > 1 << 26:
            x = torch.randint(-128, 127, (M, K), dtype=torch.int8, device=dev)
            y = torch.randint(-128, 127, (N, K), dtype=torch.int8, device=dev)
            dist.broadcast(x, 0)
            dist.broadcast(y, 0)
        else:
            x = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=gen).to(dev)
            y = torch.randint(-128, 127, (N, K), dtype=torch.int8, generator=gen).to(dev)
        KB, NB = -(-K // 128), -(-N // 128)
        sa = (torch.rand(M, KB, generator=gen) * 0.02 + 1e-3).to(dev)
        sw = (torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3).to(dev)
        y_r, sw_r = gdist.shard_weight(y, sw, rank, world)
        fg = gdist.FusedGatherGemm(M, N)
        out = fg.run(x, y_r.contiguous(), sa, sw_r.contiguous())
        torch.cuda.synchronize()
        if M * N <= 1 << 26:
            ref = g.matmul_blockwise(x, y, sa, sw)
            same = torch.equal(out.view(torch.int16), ref.view(torch.int16))
        else:  # sampled rows against the unsharded kernel on a row slice
            rows = torch.arange(0, M, 997, device=dev)
            ref = g.matmul_blockwise(x[rows].contiguous(), y, sa[rows].contiguous(), sw)
            same = torch.equal(out[rows].view(torch.int16), ref.view(torch.int16))
        ok = ok and same
        msg = f"rank {rank}: fused gather {M}x{N}x{K} world {world}: bit-equal to the unsharded kernel = {same}"
        if timed:
            ts = []
            for _ in range(5):
                dist.barrier()
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fg.run(x, y_r, sa, sw_r)
                e.record()
                torch.cuda.synchronize()
                ts.append(s.elapsed_time(e))
            t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            slices = None
            tn = []
            for _ in range(5):
                dist.barrier()
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                local = g.matmul_blockwise(x, y_r, sa, sw_r)
                slices = gdist.all_gather_slices(local, slices)
                e.record()
                torch.cuda.synchronize()
                tn.append(s.elapsed_time(e))
            t2 = torch.tensor([sorted(tn)[len(tn) // 2]], device=dev)
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
            msg += f" | fused {t.item():.3f} ms, GEMM + NCCL all-gather {t2.item():.3f} ms (max over ranks)"
        print(msg, flush=True)
        fg.close()
    # K-sharded (row-parallel) form: every rank holds a K slice, the fp32 partials cross NVLink in one all-to-all and
    # are added in rank order; compared with the same sum computed on this GPU alone from all slices.
    M, N, K = 64 * world, 1024, 2048
    gen = torch.Generator().manual_seed(4321)
    x = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=gen).to(dev)
    y = torch.randint(-128, 127, (N, K), dtype=torch.int8, generator=gen).to(dev)
    sa = (torch.rand(M, K // 128, generator=gen) * 0.02 + 1e-3).to(dev)
    sw = (torch.rand(N // 128, K // 128, generator=gen) * 0.02 + 1e-3).to(dev)

    def k_slice(r):
        k0, k1 = gdist.kshard_bounds(K, world, r)
        return (x[:, k0:k1].contiguous(), y[:, k0:k1].contiguous(), sa[:, k0 // 128:k1 // 128].contiguous(),
                sw[:, k0 // 128:k1 // 128].contiguous())

    rows = gdist.matmul_blockwise_ksharded(*k_slice(rank))
    alone = g.sum_parts_bf16(torch.stack([g.matmul_blockwise_f32(*k_slice(r)) for r in range(world)]))
    m = M // world
    same = torch.equal(rows.view(torch.int16), alone[rank * m:(rank + 1) * m].view(torch.int16))
    ok = ok and same
    print(f"rank {rank}: k-sharded reduce-scatter {M}x{N}x{K} world {world}: bit-equal to the single-GPU sum = {same}", flush=True)
    # the same with the data movement fused into the GEMM epilogue (peer stores of fp32 row blocks), twice in a row
    # (the two receive areas alternate)
    frs = gdist.FusedReduceScatterGemm(M, N)
    for it in range(2):
        rows2 = frs.run(*k_slice(rank))
        same2 = torch.equal(rows2.view(torch.int16), alone[rank * m:(rank + 1) * m].view(torch.int16))
        ok = ok and same2
        print(f"rank {rank}: fused reduce-scatter call {it}: bit-equal to the single-GPU sum = {same2}", flush=True)
    frs.close()
    # timing of both forms on a larger row-parallel shape (K = 8192 in all, sharded; device time, max over ranks)
    Mt, Nt, Kt = 4096, 8192, 8192 // world
    xt = torch.randint(-128, 127, (Mt, Kt), dtype=torch.int8, device=dev)
    yt = torch.randint(-128, 127, (Nt, Kt), dtype=torch.int8, device=dev)
    sat = torch.rand(Mt, Kt // 128, device=dev) * 0.02 + 1e-3
    swt = torch.rand(Nt // 128, Kt // 128, device=dev) * 0.02 + 1e-3
    frs = gdist.FusedReduceScatterGemm(Mt, Nt)

    def timed(fn):
        ts = []
        for _ in range(6):
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        t = torch.tensor([sorted(ts[1:])[len(ts[1:]) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    t_fused = timed(lambda: frs.run(xt, yt, sat, swt))
    t_nccl = timed(lambda: gdist.matmul_blockwise_ksharded(xt, yt, sat, swt))
    same3 = torch.equal(frs.run(xt, yt, sat, swt).view(torch.int16), gdist.matmul_blockwise_ksharded(xt, yt, sat, swt).view(torch.int16))
    ok = ok and same3
    if rank == 0:
        print(f"k-sharded {Mt}x{Nt}x{Kt * world} over {world} ranks: fused reduce-scatter {t_fused:.3f} ms, GEMM + NCCL all-to-all + sum "
              f"{t_nccl:.3f} ms (max over ranks); results identical = {same3}", flush=True)
    frs.close()
    st = g.device_status()
    print(f"rank {rank}: kernel status {st}", flush=True)
    dist.destroy_process_group()
    return 0 if ok and st == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
