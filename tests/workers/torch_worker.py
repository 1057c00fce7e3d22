"""One rank of the process-group test: torch.distributed collectives through backend "dccl" on CPU
tensors (and on CUDA tensors when --cuda), checked against values computed from the ranks' seeds."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import dccl_b200.parallel.process_group  # noqa: E402,F401  (registers the backend)


def tensor_for(rank, n, dtype, dev):
    g = torch.Generator().manual_seed(1234 + rank)
    if dtype in (torch.int32, torch.int64):
        return torch.randint(-1000, 1000, (n,), generator=g, dtype=dtype).to(dev)
    return (torch.rand(n, generator=g) * 2 - 1).to(dtype).to(dev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--ddp", action="store_true")
    ap.add_argument("--extra", action="store_true", help="all-to-all / gather / scatter, list forms, batch_isend_irecv, objects, subgroups")
    args = ap.parse_args()
    rank, world = int(os.environ["DCCL_RANK"]), int(os.environ["DCCL_WORLD_SIZE"])
    port = int(os.environ["DCCL_MASTER_PORT"]) + 1
    if args.cuda:
        torch.cuda.set_device(int(os.environ.get("DCCL_LOCAL_DEVICE", "0")))
    dev = torch.device("cuda", torch.cuda.current_device()) if args.cuda else torch.device("cpu")
    dist.init_process_group("dccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    fails = []

    def check(ok, what):
        if not ok:
            fails.append(what)

    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.float64):
        for n in (1, 1000, 70001):
            ins = [tensor_for(r, n, dtype, dev) for r in range(world)]
            tol = dict(rtol=2e-2, atol=2e-2 * world) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
            want = torch.stack([x.double() for x in ins]).sum(0)
            t = ins[rank].clone()
            dist.all_reduce(t)
            check(torch.allclose(t.double(), want, **tol), "all_reduce %s %d" % (dtype, n))
            t = ins[rank].clone()
            w = dist.all_reduce(t, op=dist.ReduceOp.MAX, async_op=True)
            w.wait()
            check(torch.equal(t, torch.stack(ins).max(0).values), "all_reduce max async %s %d" % (dtype, n))
            if dtype.is_floating_point:
                t = ins[rank].clone()
                dist.all_reduce(t, op=dist.ReduceOp.AVG)
                check(torch.allclose(t.double(), want / world, **tol), "all_reduce avg %s %d" % (dtype, n))
            for root in {0, world - 1}:
                t = ins[rank].clone()
                dist.broadcast(t, src=root)
                check(torch.equal(t, ins[root]), "broadcast %s %d root %d" % (dtype, n, root))
                t = ins[rank].clone()
                dist.reduce(t, dst=root)
                check(rank != root or torch.allclose(t.double(), want, **tol), "reduce %s %d root %d" % (dtype, n, root))
            out = torch.empty(n * world, dtype=dtype, device=dev)
            dist.all_gather_into_tensor(out, ins[rank])
            check(torch.equal(out, torch.cat(ins)), "all_gather_into_tensor %s %d" % (dtype, n))
            lst = [torch.empty(n, dtype=dtype, device=dev) for _ in range(world)]
            dist.all_gather(lst, ins[rank])
            check(all(torch.equal(a, b) for a, b in zip(lst, ins)), "all_gather %s %d" % (dtype, n))
            big = [tensor_for(100 + r, n * world, dtype, dev) for r in range(world)]
            wantrs = torch.stack([x.double() for x in big]).sum(0)[rank * n:(rank + 1) * n]
            out = torch.empty(n, dtype=dtype, device=dev)
            dist.reduce_scatter_tensor(out, big[rank])
            check(torch.allclose(out.double(), wantrs, **tol), "reduce_scatter_tensor %s %d" % (dtype, n))
    if args.extra:
        # all-to-all, gather, scatter (grouped send / recv underneath)
        for dtype in (torch.float32, torch.int64):
            for n in (1, 257, 300001):
                ins = [tensor_for(200 + r, n * world, dtype, dev) for r in range(world)]
                out = torch.empty(n * world, dtype=dtype, device=dev)
                dist.all_to_all_single(out, ins[rank])
                want = torch.cat([ins[p][rank * n:(rank + 1) * n] for p in range(world)])
                check(torch.equal(out, want), "all_to_all_single %s %d" % (dtype, n))
                outs = [torch.empty(n, dtype=dtype, device=dev) for _ in range(world)]
                dist.all_to_all(outs, list(ins[rank].split(n)))
                check(torch.equal(torch.cat(outs), want), "all_to_all %s %d" % (dtype, n))
                for root in {0, world - 1}:
                    lst = [torch.empty(n, dtype=dtype, device=dev) for _ in range(world)] if rank == root else None
                    dist.gather(ins[rank][:n], lst, dst=root)
                    check(rank != root or all(torch.equal(lst[p], ins[p][:n]) for p in range(world)), "gather %s %d root %d" % (dtype, n, root))
                    got = torch.empty(n, dtype=dtype, device=dev)
                    dist.scatter(got, list(ins[root].split(n)) if rank == root else None, src=root)
                    check(torch.equal(got, ins[root][rank * n:(rank + 1) * n]), "scatter %s %d root %d" % (dtype, n, root))
        # uneven splits: rank r sends (p + 1) rows of 3 to rank p and receives (r + 1) rows from everybody
        rows_in = sum(p + 1 for p in range(world))
        src = (torch.arange(rows_in * 3, dtype=torch.float32) + 1000 * rank).reshape(rows_in, 3).to(dev)
        dst = torch.empty(((rank + 1) * world, 3), dtype=torch.float32, device=dev)
        dist.all_to_all_single(dst, src, output_split_sizes=[rank + 1] * world, input_split_sizes=[p + 1 for p in range(world)])
        off = sum(p + 1 for p in range(rank)) * 3
        want = torch.cat([(torch.arange(off, off + (rank + 1) * 3, dtype=torch.float32) + 1000 * p).reshape(rank + 1, 3) for p in range(world)]).to(dev)
        check(torch.equal(dst, want), "all_to_all_single with uneven splits")
    # point to point: even ranks send to the next odd rank
    if world >= 2:
        msg = torch.full((5000,), float(rank), device=dev)
        if rank % 2 == 0 and rank + 1 < world:
            dist.send(msg, rank + 1)
        elif rank % 2 == 1:
            dist.recv(msg, rank - 1)
            check(bool((msg == float(rank - 1)).all()), "send/recv")
    dist.barrier()

    if args.extra:
        # list forms: reduce_scatter from a list of tensors (goes through a temporary), product and min
        parts = [torch.full((257,), float(rank + 1 + p), device=dev) for p in range(world)]
        out = torch.empty(257, device=dev)
        dist.reduce_scatter(out, parts)
        check(bool((out == float(sum(r + 1 + rank for r in range(world)))).all()), "reduce_scatter (list)")
        t = torch.full((33,), float(rank + 1), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.PRODUCT)
        want = 1.0
        for r in range(world):
            want *= r + 1
        check(bool((t == want).all()), "all_reduce product")
        t = torch.full((33,), rank + 5, device=dev, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        check(bool((t == 5).all()), "all_reduce min")

        # batch_isend_irecv: a ring in which everybody sends first, with messages longer than a FIFO; one grouped launch
        if world >= 2:
            big = torch.full((1 << 20,), float(rank), device=dev)          # 4 MB
            got = torch.empty_like(big)
            works = dist.batch_isend_irecv([dist.P2POp(dist.isend, big, (rank + 1) % world), dist.P2POp(dist.irecv, got, (rank - 1) % world)])
            for w in works:
                w.wait()
            if args.cuda:
                torch.cuda.synchronize()
            check(bool((got == float((rank - 1) % world)).all()), "batch_isend_irecv ring")

        # Python objects ride on byte tensors: broadcast_object_list, all_gather_object
        objs = [{"from": rank, "payload": list(range(rank + 3))}]
        dist.broadcast_object_list(objs, src=world - 1, device=dev)
        check(objs[0] == {"from": world - 1, "payload": list(range(world + 2))}, "broadcast_object_list")
        gathered = [None] * world
        dist.all_gather_object(gathered, ("rank", rank))
        check(gathered == [("rank", r) for r in range(world)], "all_gather_object")

        # subgroups: every rank calls new_group, only the members get a communicator; then a second world-wide group
        if world >= 3:
            members = list(range(0, world, 2))
            evens = dist.new_group(ranks=members)
            t = torch.full((1000,), float(rank), device=dev)
            if rank in members:
                dist.all_reduce(t, group=evens)
                check(bool((t == float(sum(members))).all()), "all_reduce in a subgroup")
                out = torch.empty(len(members), device=dev)
                dist.all_gather_into_tensor(out, torch.tensor([float(rank)], device=dev), group=evens)
                check(out.tolist() == [float(m) for m in members], "all_gather in a subgroup")
            again = dist.new_group(ranks=list(range(world)))
            t = torch.full((10,), 1.0, device=dev)
            dist.all_reduce(t, group=again)
            check(bool((t == float(world)).all()), "all_reduce in a second world-wide group")
            dist.barrier()

    if args.ddp:
        # DistributedDataParallel over the backend: gradients must equal the average of the per-rank gradients
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).to(dev)
        ref = [p.detach().clone() for p in model.parameters()]
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index] if args.cuda else None, bucket_cap_mb=1)
        xs = [torch.randn(16, 32, generator=torch.Generator().manual_seed(50 + r)) for r in range(world)]
        ddp(xs[rank].to(dev)).pow(2).mean().backward()
        if args.cuda:
            torch.cuda.synchronize()
        grads = [p.grad.detach().cpu().double() for p in model.parameters()]
        # serial reference on the CPU
        want = None
        for r in range(world):
            m = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8))
            with torch.no_grad():
                for p, q in zip(m.parameters(), ref):
                    p.copy_(q.cpu())
            m(xs[r]).pow(2).mean().backward()
            g = [p.grad.double() for p in m.parameters()]
            want = g if want is None else [a + b for a, b in zip(want, g)]
        want = [w / world for w in want]
        check(all(torch.allclose(a, b, rtol=1e-4, atol=1e-6) for a, b in zip(grads, want)), "DDP gradients")

    if args.extra:
        # differential run: the same calls through a gloo group (CPU tensors) or a stock NCCL group (CUDA tensors)
        # over the same ranks
        gloo = dist.new_group(ranks=list(range(world)), backend="nccl" if args.cuda else "gloo")
        for dtype in (torch.float32, torch.int64):
            n = 4099
            mine = tensor_for(300 + rank, n * world, dtype, dev)
            a, b = mine.clone(), mine.clone()
            dist.all_reduce(a)
            dist.all_reduce(b, group=gloo)
            check(torch.allclose(a.double(), b.double(), rtol=1e-5, atol=1e-5), "all_reduce against the other library %s" % dtype)
            a, b = mine.clone(), mine.clone()
            dist.all_reduce(a, op=dist.ReduceOp.MIN)
            dist.all_reduce(b, op=dist.ReduceOp.MIN, group=gloo)
            check(torch.equal(a, b), "all_reduce min against the other library %s" % dtype)
            a, b = mine.clone(), mine.clone()
            dist.broadcast(a, src=world - 1)
            dist.broadcast(b, src=world - 1, group=gloo)
            check(torch.equal(a, b), "broadcast against the other library %s" % dtype)
            a, b = mine.clone(), mine.clone()
            dist.reduce(a, dst=0)
            dist.reduce(b, dst=0, group=gloo)
            check(rank != 0 or torch.allclose(a.double(), b.double(), rtol=1e-5, atol=1e-5), "reduce against the other library %s" % dtype)
            la = [torch.empty_like(mine) for _ in range(world)]
            lb = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(la, mine)
            dist.all_gather(lb, mine, group=gloo)
            check(all(torch.equal(x, y) for x, y in zip(la, lb)), "all_gather against the other library %s" % dtype)
            a, b = torch.empty_like(mine), torch.empty_like(mine)
            dist.all_to_all_single(a, mine)
            dist.all_to_all_single(b, mine, group=gloo)
            check(torch.equal(a, b), "all_to_all_single against the other library %s" % dtype)
        if args.cuda:
            torch.cuda.synchronize()
        dist.barrier()

    dist.destroy_process_group()
    if fails:
        print("FAILED on rank %d: %s" % (rank, "; ".join(fails[:10])))
        sys.exit(1)
    print("OK")


if __name__ == "__main__":
    main()
