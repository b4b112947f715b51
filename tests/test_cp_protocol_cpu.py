"""Context-parallel hop protocol with CPU ranks (gloo, world size 2 and 3): the boundary-state chain of
palimpsa_b200.parallel, with the float64 oracle standing in for the CUDA kernels.  Also the failure
path: a rank that dies before sending makes its neighbour's receive end with an error, not a hang."""
import datetime
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=180):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _cp_worker(rank, world, port, q_out):
    try:
        _init(rank, world, port)
        from oracle import palimpsa_oracle as orc
        from palimpsa_b200.parallel import chain_down, chain_up, shard_bounds
        torch.set_num_threads(1)
        B, T, H, K, V = 2, 45, 2, 4, 6
        d = orc.make_inputs(11, B=B, T=T, H=H, K=K, V=V, dtype=torch.float64)
        d["gt"] = d["gt"] * 0.2
        lo, hi = shard_bounds(T, rank, world)
        sl = {n: (x[:, lo:hi] if x.dim() >= 3 else x) for n, x in d.items()}
        ipb = d["Ip"].double().view(1, H, 1, 1)
        like = torch.empty(2, B, H, V, K, dtype=torch.float64)
        # ---- forward: local summary, then the chain, then the local heavy pass from the true start state
        SM, SJ, P = orc.segment_summary(sl["k"], sl["v"], sl["b"], sl["gt"], sl["g"])
        box = {}

        def local_fwd(inc):
            start = torch.zeros_like(like) if inc is None else inc
            box["start"] = start
            pb = P.view(B, H, 1, 1)
            return torch.stack([pb * start[0] + SM, pb * start[1] + SJ])

        chain_down(rank, world, None, local_fwd, like)
        M0, J0 = box["start"]
        I0 = J0 + ipb
        o, _, mu, I = orc.oracle_forward(sl["q"], sl["k"], sl["v"], sl["b"], sl["gt"], sl["g"], sl["Ip"], M0 / I0, I0)
        # ---- backward: state gradients travel up the ranks
        res = {}

        def local_bwd(inc):
            cm, ci = (None, None) if inc is None else (inc[0], inc[1])
            r = orc.oracle_backward_explicit(sl["q"], sl["k"], sl["v"], sl["b"], sl["gt"], sl["g"], sl["Ip"], sl["do"],
                                             None, M0 / I0, I0, carry_M=cm, carry_I=ci)
            res.update(r)
            return torch.stack([r["dM0"], r["dI0"]])

        chain_up(rank, world, None, local_bwd, like)
        # explicit-start ranks must not add the prior-start term to dIp; rank 0 starts from the prior
        if rank == 0:
            res["dIp"] = res["dIp"] + res["dI0"].sum((0, 2, 3))
        pg = torch.stack([res["dg"], res["dIp"]])
        dist.all_reduce(pg)
        # results travel as numpy arrays (pickled bytes): torch tensors would be passed as shared-memory handles
        # that die with this process if the parent has not opened them yet
        q_out.put((rank, lo, hi, o.numpy(), {n: res[n].numpy() for n in ("dq", "dk", "dv", "db", "dgt")}, pg.numpy(),
                   mu.numpy(), I.numpy()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        q_out.put((rank, "error", traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 3])
def test_cp_chain_matches_single_process(world):
    from oracle import palimpsa_oracle as orc
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cp_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q_out.get(timeout=400) for _ in range(world)]
    for p in procs:
        p.join(60)
    for g in got:
        assert g[1] != "error", g[2]
    got.sort(key=lambda x: x[0])
    tt = torch.from_numpy
    got = [(g[0], g[1], g[2], tt(g[3]), {n: tt(x) for n, x in g[4].items()}, tt(g[5]), tt(g[6]), tt(g[7])) for g in got]
    B, T, H, K, V = 2, 45, 2, 4, 6
    d = orc.make_inputs(11, B=B, T=T, H=H, K=K, V=V, dtype=torch.float64)
    d["gt"] = d["gt"] * 0.2
    ref = orc.oracle_fwd_bwd(d["q"], d["k"], d["v"], d["b"], d["gt"], d["g"], d["Ip"], d["do"])
    o = torch.cat([g[3] for g in got], 1)
    assert orc.rel_err(o, ref["o"]) < 1e-12
    for n in ("dq", "dk", "dv", "db", "dgt"):
        assert orc.rel_err(torch.cat([g[4][n] for g in got], 1), ref[n]) < 1e-11, n
    for g in got:
        assert orc.rel_err(g[5][0], ref["dg"]) < 1e-11 and orc.rel_err(g[5][1], ref["dIp"]) < 1e-11
    assert orc.rel_err(got[-1][6], ref["final_mu"]) < 1e-12 and orc.rel_err(got[-1][7], ref["final_I"]) < 1e-12


def _fail_worker(rank, world, port, q_out):
    try:
        _init(rank, world, port)       # generous rendezvous: the ranks' start-up times differ under load
        from palimpsa_b200.parallel import chain_down
        short = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=4))
        like = torch.zeros(2, 1, 1, 2, 2, dtype=torch.float64)

        def local(inc):
            if rank == 0:
                raise RuntimeError("rank 0 fails before it sends its boundary state")
            return like

        try:
            chain_down(rank, world, short, local, like)
            q_out.put((rank, "finished"))
        except Exception as e:  # noqa: BLE001
            q_out.put((rank, "raised", type(e).__name__, str(e)[:200]))
    except Exception:
        q_out.put((rank, "error", traceback.format_exc()))
    finally:
        q_out.close()
        q_out.join_thread()
        os._exit(0)   # a broken group cannot be torn down cleanly; leave without the atexit hooks


def test_cp_peer_failure_surfaces_as_error_not_hang():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fail_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted([q_out.get(timeout=400) for _ in range(2)], key=lambda x: x[0])
    for p in procs:
        p.join(60)
    assert got[0][1] == "raised" and "fails before" in got[0][3]
    assert got[1][1] == "raised", got[1]          # the receiver saw a timeout / connection error


def test_shard_bounds_cover_everything():
    from palimpsa_b200.parallel import shard_bounds
    for n in (1, 7, 48, 131072):
        for w in (1, 2, 3, 8):
            b = [shard_bounds(n, r, w) for r in range(w)]
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
            assert max(h - l for l, h in b) - min(h - l for l, h in b) <= 1
