"""One rank of the multi-GPU ProcessGroupB200 checks (child of test_pg_b200_gpu_multi.py)."""
import argparse
import json
import os
import sys
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
from torch.distributed.distributed_c10d import AllgatherOptions, AllToAllOptions, ReduceOp, ReduceScatterOptions


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--world", type=int, required=True)
    ap.add_argument("--store", required=True)
    a = ap.parse_args()
    torch.cuda.set_device(a.rank)
    dev = torch.device("cuda", a.rank)

    from torchft_b200.checkpointing.pg_transport import PGTransport
    from torchft_b200.collectives import allreduce_quantized
    from torchft_b200.parallel.team import ProcessGroupB200

    r, W = a.rank, a.world
    # small windows so that the chunked paths run too
    pg = ProcessGroupB200(timeout=timedelta(seconds=20), arena_bytes=8 << 20, staging_bytes=1 << 20, p2p_bytes=1 << 20)
    pg.configure(f"{a.store}/torchft/3/0", "rep", r, W)
    checks = {}

    def val(p, n, dtype=torch.float32):
        return (torch.arange(n, device=dev, dtype=torch.float32) % 97 + 100 * (p + 1)).to(dtype)

    for n in (5, 1000, 700_001):  # ragged, small (one-shot), chunked
        for dtype in (torch.float32, torch.bfloat16):
            t = val(r, n, dtype)
            pg.allreduce([t], ReduceOp.SUM).wait()
            want = sum(val(p, n, dtype).float() for p in range(W))
            checks[f"allreduce_{n}_{dtype}"] = bool(torch.allclose(t.float(), want, rtol=2e-2))
    t = val(r, 1000)
    pg.allreduce([t], ReduceOp.AVG).wait()
    checks["allreduce_avg"] = bool(torch.allclose(t, sum(val(p, 1000) for p in range(W)) / W, rtol=1e-5))

    for n, dtype in ((7, torch.int64), (4096, torch.bfloat16), (300_003, torch.float32)):
        inp = val(r, n, dtype)
        out = torch.empty(W * n, dtype=dtype, device=dev)
        pg.allgather_into_tensor_coalesced([out], [inp], AllgatherOptions()).wait()
        checks[f"allgather_into_{n}"] = all(torch.equal(out[p * n:(p + 1) * n], val(p, n, dtype)) for p in range(W))
        outs = [torch.empty(n, dtype=dtype, device=dev) for _ in range(W)]
        pg.allgather([outs], [inp], AllgatherOptions()).wait()
        checks[f"allgather_{n}"] = all(torch.equal(outs[p], val(p, n, dtype)) for p in range(W))
        b = val(r, n, dtype)
        pg.broadcast_one(b, W - 1).wait()
        checks[f"broadcast_{n}"] = bool(torch.equal(b, val(W - 1, n, dtype)))

    for chunk in (3, 1024, 200_000):
        inp = torch.cat([val(r, chunk) + 1000 * p for p in range(W)])  # chunk p goes to rank p
        out = torch.empty_like(inp)
        pg.alltoall_base(out, inp, [], [], AllToAllOptions()).wait()
        checks[f"alltoall_{chunk}"] = all(
            torch.equal(out[p * chunk:(p + 1) * chunk], val(p, chunk) + 1000 * r) for p in range(W))

    for shard, dtype in ((6, torch.float32), (4096, torch.bfloat16), (150_001, torch.float32)):
        inp = torch.cat([val(r, shard, dtype) + p for p in range(W)])
        out = torch.empty(shard, dtype=dtype, device=dev)
        opts = ReduceScatterOptions()
        pg.reduce_scatter_tensor_coalesced([out], [inp], opts).wait()
        want = sum((val(p, shard, dtype) + r).float() for p in range(W))
        checks[f"reduce_scatter_{shard}"] = bool(torch.allclose(out.float(), want, rtol=2e-2))
    out = torch.empty(8, device=dev)
    pg.reduce_scatter([out], [[val(r, 8) + p for p in range(W)]], ReduceScatterOptions()).wait()
    checks["reduce_scatter_lists"] = bool(torch.allclose(out, sum(val(p, 8) + r for p in range(W))))

    # point to point: a ring, even ranks send first
    nxt, prv = (r + 1) % W, (r - 1) % W
    for n in (1, 33, 600_000):
        got = torch.zeros(n, device=dev)
        if r % 2 == 0:
            pg.send([val(r, n)], nxt, 0).wait()
            pg.recv([got], prv, 0).wait()
        else:
            pg.recv([got], prv, 0).wait()
            pg.send([val(r, n)], nxt, 0).wait()
        checks[f"sendrecv_{n}"] = bool(torch.equal(got, val(prv, n)))

    # quantised allreduce through the public helper, and the checkpoint transport on this group
    t = torch.randn(128 * W * 40, device=dev, generator=torch.Generator(device=dev).manual_seed(r))
    refs = [torch.randn(128 * W * 40, device=dev, generator=torch.Generator(device=dev).manual_seed(p)) for p in range(W)]
    allreduce_quantized([t], ReduceOp.AVG, pg).wait()
    want = sum(refs) / W
    checks["allreduce_quantized"] = float(((t - want).abs().mean() / want.abs().mean()).item()) < 0.05

    from torchft_b200.collectives import allocate_reduce_scatter_output, reduce_scatter_quantized

    ins = [refs[r].clone()]
    out, total = allocate_reduce_scatter_output(ins, W)
    reduce_scatter_quantized(out, ins, ReduceOp.AVG, pg).wait()
    per = total // W
    want_slice = want[r * per:(r + 1) * per]
    checks["reduce_scatter_quantized"] = float(((out - want_slice).abs().mean() / want_slice.abs().mean()).item()) < 0.05

    transport = PGTransport(pg, timeout=timedelta(seconds=20), device=dev)
    state = {"w": val(0, 70_001), "b": val(0, 3, torch.bfloat16), "step": 11, "name": "x"}
    if r == 0:
        transport.send_checkpoint(list(range(1, W)), 11, state, timedelta(seconds=20))
        checks["pg_transport"] = True
    else:
        got = transport.recv_checkpoint(0, transport.metadata(), 11, timedelta(seconds=20))
        checks["pg_transport"] = bool(torch.equal(got["w"].to(dev), state["w"]) and torch.equal(got["b"].to(dev), state["b"])
                                      and got["step"] == 11 and got["name"] == "x")
    pg.barrier().wait()
    torch.cuda.synchronize()
    err = pg.errored()
    pg.shutdown()
    print(json.dumps({"rank": r, "errored": str(err), "checks": checks}), flush=True)


if __name__ == "__main__":
    main()
