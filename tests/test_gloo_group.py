"""World-size-2 checks on CPU with the gloo backend: the handle exchange of
`Buffer.connect()` (with the native runtime replaced by a recorder), and the
oracle run rank by rank over a real process group against the golden vectors."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.golden.make_golden import make_inputs, sha

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


class _RecorderRuntime:
    """Stands in for mooncake_b200.ep.Buffer: records what the bootstrap hands it."""

    def __init__(self, rank):
        self.rank = rank
        self.synced = None

    def p2p_enabled(self):
        return True

    def get_ipc_handle(self):
        return [self.rank * 100 + i for i in range(16)]

    def sync_nvlink_ipc_handles(self, handles, mask):
        self.synced = (handles, mask)

    def use_fast_path(self):
        return self.synced is not None


def _connect_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import warnings
    from mooncake_b200.mooncake_ep_buffer import Buffer
    b = Buffer.__new__(Buffer)
    b.rank, b.group_size, b.group, b.backend = rank, world, dist.group.WORLD, dist.group.WORLD
    b.runtime = _RecorderRuntime(rank)
    b._warned_active_ranks = False
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        b.connect()
        b.update_ep_member()  # membership refresh re-runs the exchange
    handles, mask = b.runtime.synced
    ok = (handles == [[r * 100 + i for i in range(16)] for r in range(world)]
          and mask == [1] * world
          and sum("active_ranks is only available" in str(x.message) for x in w) == 1)
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_connect_exchanges_handles_in_rank_order():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_connect_worker, args=(r, 2, 29731, q)) for r in range(2)]
    [p.start() for p in procs]
    res = sorted(q.get(timeout=120) for _ in procs)
    [p.join(60) for p in procs]
    assert res == [(0, True), (1, True)]


def _oracle_worker(rank, world, port, name, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import ep_oracle as ora
    g = torch.load(os.path.join(GOLDEN, f"{name}.pt"), weights_only=False)
    cfg = g["ranks"][0]["cfg"]
    x, idx, w = make_inputs(cfg, rank)
    # every rank contributes its own tokens; the group gathers them (variable counts)
    xs, idxs = [None] * world, [None] * world
    dist.all_gather_object(xs, x)
    dist.all_gather_object(idxs, idx)
    mine = ora.dispatch(xs, idxs, cfg["M"], cfg["E"], cfg["fp8"], arith="fallback")[rank]
    part = g["ranks"][rank]
    L = cfg["E"] // world
    ok = torch.equal(mine["recv_count"], part["recv_count"])
    ok &= torch.equal(mine["layout_range"], part["layout_range"])
    for le in range(L):
        n = int(part["recv_count"][le])
        ok &= torch.equal(mine["src_info"][le, :n], part["src_info"][le, :n])
        ok &= sha(mine["recv_x"][le, :n]) == part["recv_x_sha"][le]
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["c1_bf16", "small_fp8_uneven"])
def test_oracle_over_a_real_group_matches_golden(name):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_oracle_worker, args=(r, 2, 29741 + len(name), name, q))
             for r in range(2)]
    [p.start() for p in procs]
    res = sorted(q.get(timeout=180) for _ in procs)
    [p.join(60) for p in procs]
    assert res == [(0, True), (1, True)]


def _elastic_worker(rank, world, port, q):
    """The elastic wrapper's bootstrap over gloo (runtime replaced by the recorder),
    and the elastic oracle run on inputs every rank contributes through the group."""
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mooncake_b200.mooncake_elastic_buffer import ElasticBuffer
    from oracle import elastic_oracle as eo
    from tests.ep_harness import make_rank_inputs
    b = ElasticBuffer.__new__(ElasticBuffer)
    b.rank_idx, b.num_ranks, b.group, b.backend = rank, world, dist.group.WORLD, dist.group.WORLD
    b.runtime = _RecorderRuntime(rank)
    b._connect_native()
    b.update_ep_member()
    handles, mask = b.runtime.synced
    ok = handles == [[r * 100 + i for i in range(16)] for r in range(world)] and mask == [1] * world
    ok &= ElasticBuffer.get_buffer_size_hint(dist.group.WORLD, 64, 256, 4) == \
        2 * world * 64 * (32 + 4 * 256) + 2 * world * 64 * 48
    # every rank contributes its own tokens; all compute the same group-wide result
    E, K, M, H = 8 * world, 4, 64, 32
    x, idx, w = make_rank_inputs(5, rank, 20 + 7 * rank, H, E, K, "uniform", 3)
    xs, idxs, ws = [None] * world, [None] * world, [None] * world
    dist.all_gather_object(xs, x)
    dist.all_gather_object(idxs, idx)
    dist.all_gather_object(ws, w)
    outs = eo.elastic_dispatch(xs, idxs, ws, E, M, 2)
    mine = outs[rank]
    ns = [None] * world
    dist.all_gather_object(ns, mine["n"])
    # rows sent to every rank = rows every rank received
    L = E // world
    sent = [sum(1 for s in range(world) for t in range(idxs[s].shape[0])
                if d in eo.rank_lanes(idxs[s][t], L, E)) for d in range(world)]
    ok &= ns == sent and int(mine["psum_rank"][-1]) == sent[rank]
    comb = eo.elastic_combine([o["recv_x"] for o in outs], outs, idxs, E)[rank]
    reached = torch.tensor([len(eo.rank_lanes(idx[t], L, E)) for t in range(idx.shape[0])])
    ok &= torch.allclose(comb.float(), x.float() * reached.view(-1, 1), rtol=2e-2, atol=1e-2)
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_elastic_bootstrap_and_oracle_over_a_group():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_elastic_worker, args=(r, 2, 29733, q)) for r in range(2)]
    [p.start() for p in procs]
    res = sorted(q.get(timeout=180) for _ in procs)
    [p.join(60) for p in procs]
    assert res == [(0, True), (1, True)]
