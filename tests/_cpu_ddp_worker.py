"""Child process of the multi-process CPU tests (gloo). Usage: python _cpu_ddp_worker.py <scenario>.
RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT come from the environment. Prints `OK <scenario>` on
success; any exception makes the exit code non-zero."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flodl_b200 import nn  # noqa: E402
from flodl_b200.data import TensorDataSet  # noqa: E402
from flodl_b200.graph import FlowBuilder  # noqa: E402
from flodl_b200.parallel import comm  # noqa: E402
from flodl_b200.parallel.ddp import Ddp, DdpConfig, Trainer  # noqa: E402
from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend  # noqa: E402


def model(seed):
    torch.manual_seed(seed)
    return FlowBuilder.from_(nn.Linear(4, 16)).tag("a").through(nn.Tanh()).through(nn.Linear(16, 2)).tag("b").build()


def data(n=64):
    g = torch.Generator().manual_seed(123)
    x = torch.randn(n, 4, generator=g)
    w = torch.randn(4, 2, generator=g)
    return x, x @ w


def graph_ddp():
    rank, world = comm.rank(), comm.world_size()
    m = model(100 + rank)                      # different init per rank: setup must broadcast rank 0's
    Trainer.setup(m, None, lambda ps: nn.SGD(ps, 0.1, 0.9))
    assert m.is_distributed() and m.world_size() == world and len(m.devices()) == world
    assert m.chunk_ratios() == [1.0 / world] * world and sum(m.shard_sizes(10)) == 10
    ref = model(100)                           # what rank 0 started from
    ropt = nn.SGD(ref.parameters(), 0.1, 0.9)
    x, y = data()
    for step in range(5):
        xb, yb = x[step * 8:(step + 1) * 8], y[step * 8:(step + 1) * 8]
        out = m.forward(xb)                    # this rank's rows only
        n = out.t.shape[0]
        assert n == 8 // world
        start = rank * n
        nn.mse_loss(out, yb[start:start + n]).backward()
        m.step()
        nn.mse_loss(ref.forward(xb), yb).backward()
        ropt.step()
        ropt.zero_grad()
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p1.t.detach(), p2.t.detach(), atol=1e-5, rtol=1e-4, msg=f"{n1} differs from single-process training")
    assert m.training_step() == 5


def manual_ddp():
    rank, world = comm.rank(), comm.world_size()
    m = model(7 + rank)
    ddp = Ddp.wrap(m)
    flat0 = torch.cat([p.t.detach().reshape(-1) for p in m.parameters()])
    got = [torch.empty_like(flat0) for _ in range(world)]
    torch.distributed.all_gather(got, flat0)
    assert all(torch.equal(g, got[0]) for g in got), "wrap() must broadcast rank 0's parameters"
    for p in m.parameters():
        p.t.grad.fill_(float(rank + 1))
    ddp.all_reduce_gradients()
    mean = sum(range(1, world + 1)) / world
    assert all(torch.allclose(p.t.grad, torch.full_like(p.t.grad, mean)) for p in m.parameters())
    for p in m.parameters():
        p.t.grad.fill_(float(rank + 1))
    counts = [1 + 3 * r for r in range(world)]
    ddp.weighted_all_reduce_gradients(counts)
    want = sum((r + 1) * c for r, c in enumerate(counts)) / sum(counts)
    assert all(torch.allclose(p.t.grad, torch.full_like(p.t.grad, want)) for p in m.parameters())
    assert ddp.world_size() == world


def el_che_graph():
    rank, world = comm.rank(), comm.world_size()
    m = model(1)
    Trainer.setup_with(m, None, lambda ps: nn.SGD(ps, 0.05), DdpConfig().speed_hint(0, 2.0).max_anchor(4), scatter=False)
    assert m.has_el_che()
    st = m._ddp
    x, y = data(256)
    off = 0
    for sync in range(3):
        k = st.chunk_batches()
        assert k >= 1
        for _ in range(k):
            xb, yb = x[off:off + 4], y[off:off + 4]
            off = (off + 4) % 240
            st.begin_batch(4)
            nn.mse_loss(m.forward_impl([nn.module.Variable.wrap(xb)]), yb).backward()
        m.step()
    flat = torch.cat([p.t.detach().reshape(-1) for p in m.parameters()])
    got = [torch.empty_like(flat) for _ in range(world)]
    torch.distributed.all_gather(got, flat)
    assert all(torch.allclose(g, got[0]) for g in got), "replicas must stay identical under El Che"
    assert st.el_che.is_calibrated()


def _train_fn(m, batch):
    return nn.mse_loss(m.forward(batch[0]), batch[1])


def _builder(policy, backend, epochs=3):
    x, y = data(256)
    return (Trainer.builder(lambda dev: model(3), lambda ps: nn.SGD(ps, 0.05), _train_fn)
            .dataset(TensorDataSet(x, y)).batch_size(8).num_epochs(epochs).policy(policy).backend(backend))


def _check_state(state):
    assert state is not None and len(state.params) == 4
    m = model(3)
    with torch.no_grad():
        for p, s in zip(m.parameters(), state.params):
            p.t.copy_(s)
    x, y = data(256)
    loss = float(nn.mse_loss(m.forward(x), y).t.detach())
    base = float(nn.mse_loss(model(3).forward(x), y).t.detach())
    assert loss < 0.5 * base, (loss, base)


def run_fixed():
    h = _builder(ApplyPolicy.Cadence, AverageBackend.Nccl).anchor(4).max_anchor(4).run()
    state = h.join()
    _check_state(state)
    if comm.rank() == 0:
        ms = h.poll_metrics()
        assert [m.epoch for m in ms] == [0, 1, 2], [m.epoch for m in ms]
        assert ms[-1].avg_loss < ms[0].avg_loss


def run_cadence():
    _check_state(_builder(ApplyPolicy.Cadence, AverageBackend.Nccl).run().join())


def run_sync():
    _check_state(_builder(ApplyPolicy.Sync, AverageBackend.Nccl, 2).run().join())


def run_cpu_backend():
    _check_state(_builder(ApplyPolicy.Async, AverageBackend.Cpu).run().join())


def run_worker_failure():
    """Rank 1's train_fn raises in its second epoch: no averaging may be attempted with the dead
    rank, the survivor finishes, and join() still yields a state on every rank."""
    rank = comm.rank()
    calls = [0]

    def bad_train_fn(m, batch):
        calls[0] += 1
        if rank == 1 and calls[0] == 20:
            raise RuntimeError("injected worker failure")
        return _train_fn(m, batch)

    x, y = data(256)
    h = (Trainer.builder(lambda dev: model(3), lambda ps: nn.SGD(ps, 0.05), bad_train_fn)
         .dataset(TensorDataSet(x, y)).batch_size(8).num_epochs(3).policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl).run())
    state = h.join()
    assert state is not None and len(state.params) == 4


SCENARIOS = {f.__name__: f for f in (graph_ddp, manual_ddp, el_che_graph, run_fixed, run_cadence, run_sync, run_cpu_backend,
                                     run_worker_failure)}

if __name__ == "__main__":
    name = sys.argv[1]
    comm.init_process_group("gloo", timeout_s=20 if name == "run_worker_failure" else 120)
    SCENARIOS[name]()
    try:
        comm.barrier()
    except RuntimeError:
        # the survivor of `run_worker_failure` may have been inside an averaging collective when its peer raised; that
        # collective ends with the group's timeout and gloo then closes the pair, so no further collective can run
        if name != "run_worker_failure":
            raise
    try:
        comm.destroy_process_group()
    except RuntimeError:
        if name != "run_worker_failure":
            raise
    print(f"OK {name}")
