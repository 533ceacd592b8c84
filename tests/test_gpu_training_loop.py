"""The pieces either side of the fused step working together in one training loop on the GPU:
`StatelessModule.init` -> vmap(grad) -> `apply_gradient` (gathered gradients) -> `LRScheduler`
per batch -> `EarlyStopping` + `Checkpoint` per epoch (the shape of the reference's
examples/spirals loop).  Everything stays on the device until the loop asks for a Python bool."""

import pytest
import torch
from torch.func import grad_and_value, vmap
from torch.nn import Linear, ReLU, Sequential
from torch.nn.functional import binary_cross_entropy_with_logits

pytestmark = pytest.mark.gpu


def _spirals(n, gen, device):
    t = torch.rand(n, generator=gen, device=device) * 3.0 + 0.3
    label = (torch.rand(n, generator=gen, device=device) < 0.5).float()
    angle = t * 3.0 + label * torch.pi
    xy = torch.stack([t * torch.cos(angle), t * torch.sin(angle)], dim=1)
    return xy + 0.05 * torch.randn(n, 2, generator=gen, device=device), label[:, None]


@pytest.mark.parametrize("materialize", [True, False])
def test_ensemble_trains_freezes_and_restores(cuda, tmp_path, materialize):
    from churten_b200.checkpoint import Checkpoint, Snapshot
    from churten_b200.freeze import EarlyStopping
    from churten_b200.kernels import _C
    from churten_b200.lr_schedule import LRScheduler
    from churten_b200.optimizer import Adam
    from churten_b200.stateless import StatelessModule

    torch.manual_seed(0)
    gen = torch.Generator(device=cuda).manual_seed(0)
    n = 8
    def net():     # a factory: every replica gets its own initialisation
        return Sequential(Linear(2, 32), ReLU(), Linear(32, 32), ReLU(), Linear(32, 1)).to(cuda)

    lr = torch.tensor([3e-2, 1e-2, 3e-3, 1e-3, 3e-2, 1e-2, 1e-9, 1e-9], device=cuda)   # the last two cannot learn
    module, state = StatelessModule.init(net, Adam, num_replicas=n, init_randomness="different",
                                         optimizer_kwargs=dict(lr=lr, weight_decay=0.0))
    x, y = _spirals(512, gen, cuda)
    x_val, y_val = _spirals(256, gen, cuda)

    def loss_fn(params, buffers, xb, yb):
        return binary_cross_entropy_with_logits(module(params, buffers, xb), yb)

    grad_loss = vmap(grad_and_value(loss_fn), in_dims=(0, 0, None, None))
    val_loss = vmap(loss_fn, in_dims=(0, 0, None, None))
    sched = LRScheduler("CosineAnnealingLR", T_max=400)   # from the per-replica rate down to zero
    early = EarlyStopping(patience=3, threshold=1e-3)
    ckpt = Checkpoint(root_dir=tmp_path, verbose=False, deferred=True)

    first = last = None
    launches = _C.launch_count()
    steps = 0
    for epoch in range(25):
        for lo in range(0, 512, 128):
            grads, _ = grad_loss(state.params_dict, state.buffers_dict, x[lo:lo + 128], y[lo:lo + 128])
            Adam.apply_gradient(state, grads, materialize=materialize)
            sched(state)
            steps += 1
        with torch.no_grad():
            score = val_loss(state.params_dict, state.buffers_dict, x_val, y_val)
        first = score.clone() if first is None else first
        last = score
        ckpt(state, score)
        if bool(early(state, score)):
            break
    ckpt.flush()

    # replicas with a usable learning rate learned; the two with lr = 1e-9 were frozen early
    fast = [0, 1, 4, 5]
    assert (last[fast] < 0.5 * first[fast]).all() and (last[:6] < first[:6]).all(), (first, last)
    assert not state.active_mask[6:].any()
    assert state.optimizer_state["state_steps"][6:].max() < state.optimizer_state["state_steps"][:4].min()
    assert sched.t_[6:].max() < sched.t_[:4].min()            # their schedule clocks stopped too
    # one launch for the schedule and two or three for apply_gradient per batch; the snapshots add one per epoch
    per_batch = (_C.launch_count() - launches) / steps
    assert per_batch < (3.6 if materialize else 2.6) + 1.0, per_batch

    # the checkpoint on disk holds, per replica, the row of its best epoch
    best_epoch = early.best_epoch_.cpu()
    saved = Snapshot.from_file(tmp_path).mirror
    with torch.no_grad():
        live = state.params.clone()
        ckpt.load_best(state)
        restored_score = val_loss(state.params_dict, state.buffers_dict, x_val, y_val)
    assert torch.equal(state.params.cpu(), saved["params"])
    assert (restored_score[:6] <= last[:6] + 1e-6).all()
    assert best_epoch.shape == (n,)
    assert not torch.equal(live, state.params) or bool((best_epoch == epoch).all())
