"""DistributedOptimizer, callbacks, elastic state and checkpoint/resume on CPU ranks."""
import math
import os

import pytest
import torch

from mp_util import run_ranks


def _make(seed):
    from tips_b200.models.mnist_cnn import MnistCNN
    torch.manual_seed(seed)
    return MnistCNN()


def _dp_matches_single_process(rank, size, fused, passes):
    import tips_b200 as tips
    from tips_b200.models.mnist_cnn import synthetic_batch
    from tips_b200.ops.optim import FusedSGD
    model = _make(1234 + rank)          # different initial weights on purpose
    tips.broadcast_parameters(model.state_dict(), root_rank=0)
    ref = _make(1234)
    make = (lambda p: FusedSGD(p, lr=0.01, momentum=0.9)) if fused else (lambda p: torch.optim.SGD(p, lr=0.01, momentum=0.9))
    opt = tips.DistributedOptimizer(make(model.parameters()), named_parameters=model.named_parameters(),
                                    backward_passes_per_step=passes, fused_update=True if fused else None)
    assert type(opt).__name__ == ("FusedSGD" if fused else "SGD")  # same class name as the wrapped optimizer
    # without a symmetric window (CPU ranks) the step cannot move into the allreduce kernel: separate update
    assert not opt._tips_update_in_allreduce
    ropt = torch.optim.SGD(ref.parameters(), lr=0.01, momentum=0.9)
    for step in range(3):
        for k in range(passes):
            x, y = synthetic_batch(16, 1000 * step + 10 * k + rank)
            torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
        opt.zero_grad()
        for k in range(passes):
            xs, ys = zip(*[synthetic_batch(16, 1000 * step + 10 * k + r) for r in range(size)])
            (torch.nn.functional.cross_entropy(ref(torch.cat(xs)), torch.cat(ys)) / passes).backward()
        ropt.step()
        ropt.zero_grad()
    for (k, a), (_, b) in zip(model.state_dict().items(), ref.state_dict().items()):
        assert torch.allclose(a, b, atol=2e-5), (k, (a - b).abs().max())


@pytest.mark.parametrize("fused", [False, True])
def test_distributed_optimizer_matches_single_process(fused):
    run_ranks(_dp_matches_single_process, 2, fused, 1)


def test_backward_passes_per_step():
    run_ranks(_dp_matches_single_process, 2, False, 2)


@pytest.mark.parametrize("fused", [False, True])
def test_buckets_reduced_in_slices(fused):
    """64 KB slices cut the 4.8 MB bucket of the CNN into several collectives (a slice is a run of whole
    parameters) launched as backward goes; the trained weights still equal the single-process run, also with two
    backward passes per step."""
    run_ranks(_dp_matches_single_process, 2, fused, 2, env={"TIPS_FUSION_SLICE_BYTES": "65536"})


def _slices_are_used(rank, size):
    import tips_b200 as tips
    model = _make(3)
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01))
    b = opt._tips_buckets[0]
    assert len(b.slice_list) >= 2 and sum(c for _, _, _, c in b.slice_list) == b.numel
    assert [s[0] for s in b.slice_list[1:]] == [s[1] for s in b.slice_list[:-1]]     # consecutive parameter runs
    before = tips.metrics()["ops_enqueued"]
    from tips_b200.models.mnist_cnn import synthetic_batch
    x, y = synthetic_batch(8, rank)
    torch.nn.functional.cross_entropy(model(x), y).backward()
    opt.step()
    assert tips.metrics()["ops_enqueued"] - before == len(b.slice_list)


def _explicit_groups(rank, size):
    """`groups` as the reference defines it: an integer cuts the parameters into that many allreduce groups, a list of
    parameter lists fuses each inner list and leaves the other parameters alone; training is unchanged."""
    import tips_b200 as tips
    from tips_b200.models.mnist_cnn import synthetic_batch
    model = _make(5)
    names = dict(model.named_parameters())
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01),
                                    groups=[[names["conv1.weight"], names["conv1.bias"]], [names["fc2.weight"]]])
    sizes = sorted(len(b.params) for b in opt._tips_buckets)
    assert sizes == [1] * (len(names) - 2) + [2]
    x, y = synthetic_batch(8, rank)
    torch.nn.functional.cross_entropy(model(x), y).backward()
    opt.step()
    w = tips.allgather_object(model.fc2.weight.detach().sum().item())
    model2 = _make(5)
    opt2 = tips.DistributedOptimizer(torch.optim.SGD(model2.parameters(), lr=0.01), groups=3)
    assert 3 <= len(opt2._tips_buckets) <= 4
    torch.nn.functional.cross_entropy(model2(x), y).backward()
    opt2.step()
    assert torch.allclose(model2.fc2.weight, model.fc2.weight, atol=1e-7)
    with pytest.raises(ValueError):
        tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.01), groups=[[torch.nn.Parameter(torch.ones(1))]])
    assert all(abs(v - w[0]) < 1e-6 for v in w)


def test_explicit_allreduce_groups():
    run_ranks(_explicit_groups, 2)


def test_slice_bookkeeping():
    run_ranks(_slices_are_used, 2, env={"TIPS_FUSION_SLICE_BYTES": "65536"})


def _guards(rank, size):
    import tips_b200 as tips
    model = torch.nn.Linear(4, 2)
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1))
    model(torch.ones(3, 4)).sum().backward()
    with pytest.raises(tips.TipsError, match="not been aggregated"):
        with opt.skip_synchronize():
            opt.step()
    opt.synchronize()
    with opt.skip_synchronize():
        opt.step()
    opt.zero_grad()
    model(torch.ones(3, 4)).sum().backward()
    with pytest.raises(Exception, match="more than backward_passes_per_step"):
        model(torch.ones(3, 4)).sum().backward()
    with pytest.raises(ValueError):
        tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), op=tips.Sum, gradient_predivide_factor=2.0)


def test_optimizer_guards():
    run_ranks(_guards, 2)


def _callbacks(rank, size, tmp):
    import tips_b200 as tips
    from tips_b200 import callbacks as cb
    from tips_b200.models.mnist_cnn import synthetic_batch
    from tips_b200.trainer import fit
    model = _make(rank)
    base_lr = 0.01 * size
    opt = tips.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=base_lr, momentum=0.9))
    warm = cb.LearningRateWarmupCallback(initial_lr=base_lr, warmup_epochs=2, steps_per_epoch=4)
    sched = cb.LearningRateScheduleCallback(initial_lr=base_lr, multiplier=0.1, start_epoch=2)
    ckpt = cb.BestModelCheckpoint(os.path.join(tmp, "best-{epoch}.pt"), monitor="loss")
    cbs = [cb.BroadcastGlobalVariablesCallback(0), cb.MetricAverageCallback(), warm, sched, ckpt]
    hist = fit(model, opt, torch.nn.functional.cross_entropy, lambda e, s: synthetic_batch(8, 100 * e + 10 * s + rank),
               epochs=3, steps_per_epoch=4, callbacks=cbs)
    # warm-up: lr at the end of epoch e (last batch) = base/size * ((e + 1) * (size - 1) / warmup + 1)
    assert math.isclose(hist[0]["lr"], base_lr / size * (1.0 * (size - 1) / 2 + 1), rel_tol=1e-6)
    assert math.isclose(hist[1]["lr"], base_lr, rel_tol=1e-6)
    assert math.isclose(hist[2]["lr"], base_lr * 0.1, rel_tol=1e-6)
    assert opt.param_groups[0]["momentum"] == 0.9          # momentum correction was undone
    losses = tips.allgather_object(hist[-1]["loss"])
    assert all(abs(l - losses[0]) < 1e-9 for l in losses)   # metric averaged: identical on every rank
    w = tips.allgather_object(model.fc2.weight.detach().sum().item())
    assert all(abs(x - w[0]) < 1e-6 for x in w)             # replicas stayed in sync after the broadcast
    if rank == 0:
        assert any(f.startswith("best-") for f in os.listdir(tmp))


def test_callbacks(tmp_path):
    run_ranks(_callbacks, 2, str(tmp_path))


def _elastic_and_resume(rank, size, tmp):
    import tips_b200 as tips
    from tips_b200 import elastic
    from tips_b200.ops.optim import FusedAdam
    from tips_b200.utils.checkpoint import resume, save_checkpoint
    torch.manual_seed(rank)
    model = torch.nn.Linear(8, 4)
    opt = tips.DistributedOptimizer(FusedAdam(model.parameters(), lr=0.01))
    state = elastic.State(model, opt, samples=0)
    state.sync()
    def step():
        model(torch.ones(2, 8) * (rank + 1)).sum().backward()
        opt.step()
    step()
    state.samples = 10
    state.epoch = 1
    state.commit()
    good = model.weight.detach().clone()
    step()
    state.samples = 99
    assert not torch.equal(model.weight, good)
    state.restore()
    assert torch.equal(model.weight.detach(), good) and state.samples == 10 and state.epoch == 1
    step()                                                   # optimizer state was restored as well
    path = os.path.join(tmp, "ckpt.pt")
    wrote = save_checkpoint(path, model, opt, extra={"epoch": 5})
    assert wrote == (rank == 0)
    tips.barrier()
    ref = model.weight.detach().clone()
    with torch.no_grad():
        model.weight.add_(rank + 1.0)                        # diverge, then resume from the file
    extra = resume(path, model, opt)
    assert extra["epoch"] == 5 and torch.allclose(model.weight.detach(), ref)
    # restart: a fresh, unwrapped optimizer comes back wrapped, with the saved state, on every rank
    model2 = torch.nn.Linear(8, 4)
    opt2, extra2 = tips.load_model(path, model2, FusedAdam(model2.parameters(), lr=0.5))
    assert type(opt2).__name__ == "FusedAdam" and hasattr(opt2, "synchronize") and extra2["epoch"] == 5
    assert torch.allclose(model2.weight.detach(), ref) and opt2.param_groups[0]["lr"] == 0.01
    model2(torch.ones(2, 8) * (rank + 1)).sum().backward()
    opt2.step()
    w2 = tips.allgather_object(model2.weight.detach().clone())
    assert all(torch.equal(w, w2[0]) for w in w2)
    with pytest.raises(TypeError):          # another optimizer class than the one that wrote the file: every rank
        tips.load_model(path, model2, torch.optim.SGD(model2.parameters(), lr=0.1))
    commits = elastic.CommitStateCallback(state, batches_per_commit=2)
    n0 = state.commits
    for b in range(4):
        commits.on_batch_end(b)
    assert state.commits == n0 + 2
    ub = elastic.UpdateBatchStateCallback(state)
    ub.set_context(model, opt, {"steps": 10})
    ub.on_train_begin()
    ub.on_batch_end(3)
    assert state.batch == 4
    ub.on_epoch_begin(0)
    assert ub.params["steps"] == 6
    ue = elastic.UpdateEpochStateCallback(state)
    ue.on_train_begin()
    ue.on_epoch_end(0)                                       # first epoch of the restarted loop
    assert state.epoch == 2


def test_elastic_state_and_resume(tmp_path):
    run_ranks(_elastic_and_resume, 2, str(tmp_path))


def _elastic_retry(rank, size):
    """A step fails on the host (rank 1's request to the coordinator is dropped, so the tensor stalls on rank 0 and
    times out on rank 1); elastic.run resets the collectives, rolls back to the last commit and finishes the run
    with the weights of an undisturbed run, identical on every rank."""
    import ctypes
    import tips_b200 as tips
    from tips_b200 import _lib, elastic
    tips.set_config(collective_timeout_s=4.0)

    def make():
        torch.manual_seed(7)
        m = torch.nn.Linear(6, 3)
        return m, tips.DistributedOptimizer(torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9))

    def data(step, r):
        g = torch.Generator().manual_seed(100 * step + r)
        return torch.randn(5, 6, generator=g)

    model, opt = make()
    state = elastic.State(model, opt)
    failures = {"left": 1, "seen": 0}

    @elastic.run
    def train(state):
        for step in range(state.batch, 5):
            if step == 2 and rank == 1 and failures["left"]:
                failures["left"] = 0
                _lib.core().tips_inject_drop_requests(0, 1)
            state.model(data(step, rank)).pow(2).sum().backward()
            try:
                state.optimizer.step()
            except tips.TipsError:
                failures["seen"] += 1
                raise
            state.optimizer.zero_grad()
            state.batch = step + 1
            state.commit()

    train(state)
    assert failures["seen"] == 1 and state.batch == 5
    # an undisturbed single-process run over both ranks' data
    torch.manual_seed(7)
    ref = torch.nn.Linear(6, 3)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    for step in range(5):
        (sum(ref(data(step, r)).pow(2).sum() for r in range(size)) / size).backward()
        ropt.step()
        ropt.zero_grad()
    assert torch.allclose(model.weight.detach(), ref.weight.detach(), atol=1e-5)
    ws = tips.allgather_object(model.weight.detach().clone())
    assert all(torch.equal(w, ws[0]) for w in ws)


def test_elastic_run_retries_a_failed_step():
    run_ranks(_elastic_retry, 2, env={"TIPS_STALL_ABORT_MS": "1500", "TIPS_STALL_WARN_MS": "500"})


def _peer_loss(rank, size):
    """A rank that leaves: the others get an error on their next collective instead of hanging."""
    import os as _os
    import time
    import tips_b200 as tips
    assert tips.allreduce(torch.ones(2), op=tips.Sum)[0] == size
    if rank == size - 1:
        _os._exit(0)  # dies between steps, nothing in flight
    time.sleep(1.0)
    with pytest.raises(tips.TipsError):
        tips.allreduce(torch.ones(2), op=tips.Sum, name="after_loss")
    _os._exit(0)


def test_rank_loss_is_an_error_not_a_hang():
    run_ranks(_peer_loss, 3, env={"TIPS_STALL_ABORT_MS": "3000", "TIPS_HOST_TIMEOUT_MS": "5000"})


def _fit_with_lr_schedule(rank, size):
    """The reference's Keras integration test: fit for 10 steps with Adam, an exponential learning-rate decay, the
    distributed optimizer and the initial broadcast (tips/tensorflow/test_tensorflow2_keras.py:28-52); here the decay
    is a stock torch scheduler driving the wrapped optimizer, and the replicas must end identical."""
    import tips_b200 as tips
    from tips_b200 import callbacks as cb
    from tips_b200.trainer import fit
    torch.manual_seed(rank)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    opt = tips.DistributedOptimizer(torch.optim.Adam(model.parameters(), lr=0.01 * size))
    sched = torch.optim.lr_scheduler.ExponentialLR(opt, gamma=0.9)

    def batches(epoch, step):
        g = torch.Generator().manual_seed(100 * epoch + step * size + rank)
        return torch.randn(8, 8, generator=g), torch.randint(0, 4, (8,), generator=g)

    class StepSchedule(cb.Callback):
        def on_epoch_end(self, epoch, logs=None):
            sched.step()

    history = fit(model, opt, torch.nn.functional.cross_entropy, batches, 2, 5,
                  [cb.BroadcastGlobalVariablesCallback(0), cb.MetricAverageCallback(), StepSchedule()], verbose=0)
    assert len(history) == 2 and abs(opt.param_groups[0]["lr"] - 0.01 * size * 0.81) < 1e-9
    weights = tips.allgather_object(model[0].weight.detach().clone())
    assert all(torch.equal(weights[0], w) for w in weights)
    losses = tips.allgather_object(history[-1]["loss"])
    assert all(abs(losses[0] - v) < 1e-9 for v in losses)        # averaged metric: the same number everywhere


def test_fit_with_a_torch_lr_scheduler():
    run_ranks(_fit_with_lr_schedule, 2)



def _gradient_tape(rank, size):
    """tape.gradient returns the ranks' gradients averaged (or summed), whatever the grouping, the wire format or
    the kind of gradient; a parameter the loss does not touch gives None."""
    import tips_b200 as tips
    torch.manual_seed(0)
    emb = torch.nn.Embedding(20, 4, sparse=True)
    lin = torch.nn.Linear(4, 3)
    unused = torch.nn.Parameter(torch.zeros(2))
    hook = tips.BroadcastGlobalVariablesHook(0, torch.nn.ModuleList([emb, lin]))
    hook.begin()
    hook()                                                    # second call: nothing happens
    params = [emb.weight, lin.weight, lin.bias, unused]

    def loss_of(r):
        ids = torch.tensor([r, r + 1, 7, 7])
        return (lin(emb(ids)) * (r + 1.0)).pow(2).sum()

    def local(r):
        g = torch.autograd.grad(loss_of(r), params, allow_unused=True)
        return [None if x is None else (x.to_dense() if x.is_sparse else x) for x in g]

    every = [local(r) for r in range(size)]
    mean = [None if every[0][i] is None else sum(e[i] for e in every) / size for i in range(len(params))]
    total = [None if m is None else m * size for m in mean]

    def check(got, want, tol=1e-6):
        assert got[3] is None
        for g, w in zip(got[:3], want[:3]):
            g = g.to_dense() if g.is_sparse else g
            assert torch.allclose(g, w, atol=tol, rtol=tol), (g - w).abs().max()

    with tips.DistributedGradientTape() as tape:
        loss = loss_of(rank)
    got = tape.gradient(loss, params)
    assert got[0].is_sparse                                   # travelled as two allgathers
    check(got, mean)
    for kwargs in ({"sparse_as_dense": True, "groups": 2}, {"sparse_as_dense": True, "groups": [[lin.weight, lin.bias]]},
                   {"sparse_as_dense": True, "op": tips.Sum}, {"sparse_as_dense": True, "gradient_predivide_factor": 2.0},
                   {"sparse_as_dense": True, "groups": 1, "compression": tips.Compression.fp16}):
        with tips.DistributedGradientTape(name="tape." + "_".join(sorted(kwargs)), **kwargs) as tape:
            loss = loss_of(rank)
        got = tape.gradient(loss, params)
        assert not got[0].is_sparse
        check(got, total if kwargs.get("op") == tips.Sum else mean, 5e-2 if "compression" in kwargs else 1e-5)
    with tips.DistributedGradientTape(persistent=True, sparse_as_dense=True) as tape:
        loss = loss_of(rank)
    check(tape.gradient(loss, params), mean)
    check(tape.gradient(loss, params), mean)                  # the graph was kept
    with pytest.raises(ValueError):
        tips.DistributedGradientTape(op=tips.Sum, gradient_predivide_factor=2.0)
    with pytest.raises(ValueError):
        tips.DistributedGradientTape(groups=0)
    assert int(tips.local_size_op()) == tips.local_size() and int(tips.local_rank_op()) == tips.local_rank()


def test_distributed_gradient_tape():
    run_ranks(_gradient_tape, 3)
