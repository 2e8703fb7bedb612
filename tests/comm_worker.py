"""Child process of tests/test_comm_gpu.py: one rank of a 2-GPU run of the gradient exchange (he_comm_*).
Launched by torch.distributed.run; the unique id travels over a gloo (CPU) process group, the gradients
over the library's own NCCL communicator.  Exit code 0 = the scenario behaved as expected."""
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import helium_b200 as hb  # noqa: E402


def main():
    scenario = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    ctx = hb.Context(local)

    def exchange(b: bytes) -> bytes:
        t = torch.tensor(list(b), dtype=torch.uint8)
        dist.broadcast(t, src=0)
        return bytes(t.tolist())

    if scenario == "never_joins":
        # rank 1 leaves before it ever creates its communicator (no kernel or collective of its own in
        # flight); rank 0's creation must end at its deadline with the communicator aborted
        if rank == 1:
            exchange(b"\0" * 128)
            dist.destroy_process_group()
            return 0
        t0 = time.perf_counter()
        try:
            hb.Comm(ctx, rank, world, exchange, timeout_ms=3000)
        except hb.HeliumError as e:
            dt = time.perf_counter() - t0
            assert e.status == -7, (e.status, e.message)
            assert 2.5 < dt < 30.0, dt
            print("rank 0: creation gave up after %.1f s: %s" % (dt, e.message))
            return 0
        raise AssertionError("he_comm_create returned although rank 1 never joined")

    comm = hb.Comm(ctx, rank, world, exchange, max_ctas=8, timeout_ms=30000)
    dev = torch.device("cuda", local)
    if scenario == "allreduce":
        r = np.random.default_rng(100 + rank)
        a = r.standard_normal(1 << 20).astype(np.float32)
        b = r.standard_normal(4097).astype(np.float32)
        ta = torch.from_numpy(a).to(dev).to(torch.bfloat16)
        tb = torch.from_numpy(b).to(dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        for _ in range(3):                               # same layout thrice: the layout check runs once
            ta2, tb2 = ta.clone(), tb.clone()
            side.wait_stream(torch.cuda.current_stream())
            comm.allreduce([ta2], mean=True, stream=side)
            comm.allreduce([tb2], mean=False, stream=side)
        side.synchronize()
        comm.poll()
        # expected values from both ranks' seeds
        ra, rb = [], []
        for k in range(world):
            rr = np.random.default_rng(100 + k)
            ra.append(torch.from_numpy(rr.standard_normal(1 << 20).astype(np.float32)).to(torch.bfloat16).float().numpy())
            rb.append(rr.standard_normal(4097).astype(np.float32))
        want_a = np.mean(ra, axis=0)
        want_b = np.sum(rb, axis=0)
        got_a = ta2.float().cpu().numpy()
        got_b = tb2.cpu().numpy()
        assert np.allclose(got_a, want_a, rtol=1e-2, atol=1e-2), float(np.abs(got_a - want_a).max())
        assert np.allclose(got_b, want_b, rtol=1e-6, atol=1e-6), float(np.abs(got_b - want_b).max())
    elif scenario == "layout_mismatch":
        n = 1024 if rank == 0 else 2048
        t = torch.ones(2048, dtype=torch.float32, device=dev)
        try:
            comm.allreduce([t[:n]], mean=False)
        except hb.HeliumError as e:
            assert e.status == -1 and "different bucket layout" in e.message, (e.status, e.message)
            torch.cuda.synchronize()
            assert float(t.sum().item()) == 2048.0       # nothing was reduced
            # the communicator is still healthy: an agreed layout goes through
            comm.allreduce([t], mean=False)
            torch.cuda.synchronize()
            assert float(t[0].item()) == float(world)
        else:
            raise AssertionError("mismatched layouts were accepted")
    else:
        raise SystemExit("unknown scenario " + scenario)
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank}: {scenario} ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
