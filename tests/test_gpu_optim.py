"""GPU: the fused clip + AdamW step (csrc/optim.cu, jetfire_int8training_b200.optim.ClipAdamW) against
torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW (the reference's optimiser step, INT8_GPT2/train.py:320-329).
Floating point: parameters within rtol 2e-6 / atol 1e-7 after every step (same fp32 expressions; the global norm is summed in a
different order), the reported norm within 1e-5 relative."""
import pytest
import torch

from gpu_util import DEV

pytestmark = pytest.mark.gpu


def _make(shapes, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter((0.05 * torch.randn(*s, generator=g)).to(DEV)) for s in shapes]


@pytest.mark.parametrize("case", ["few", "many", "noclip"])
def test_clip_adamw_matches_torch(case):
    from jetfire_int8training_b200.optim import ClipAdamW
    if case == "many":        # more tensors than one launch takes (160), sizes that are not multiples of the 4096-element chunk
        shapes = [(36,), (4100,), (64, 68)] * 60 + [(300, 1000)]
    else:
        shapes = [(768,), (2304, 768), (768, 768), (4,), (50304, 64), (3072, 768)]
    max_norm = 0.0 if case == "noclip" else 1.0
    ours, ref = _make(shapes, 1), _make(shapes, 1)
    groups = lambda ps: [([p for p in ps if p.dim() >= 2], 0.1), ([p for p in ps if p.dim() < 2], 0.0)]
    opt = ClipAdamW(groups(ours), lr=6e-4, betas=(0.9, 0.95), eps=1e-8, max_norm=max_norm)
    topt = torch.optim.AdamW([{"params": g, "weight_decay": wd} for g, wd in groups(ref)], lr=6e-4, betas=(0.9, 0.95), eps=1e-8)
    gen = torch.Generator().manual_seed(2)
    for step in range(4):
        scale = 10.0 if step % 2 == 0 else 1e-3          # a step that is clipped and one that is not
        for a, b in zip(ours, ref):
            gr = (scale * torch.randn(a.shape, generator=gen)).to(DEV)
            a.grad = gr.clone(); b.grad = gr.clone()
        versions = [p._version for p in ours]
        out = opt.step()
        tn = torch.nn.utils.clip_grad_norm_(ref, max_norm) if max_norm > 0 else torch.nn.utils.get_total_norm([p.grad for p in ref])
        topt.step()
        assert abs(float(out[0]) - float(tn)) <= 1e-5 * float(tn)
        want = min(1.0, max_norm / (float(tn) + 1e-6)) if max_norm > 0 else 1.0
        assert abs(float(out[1]) - want) <= 1e-5 * want
        for a, b in zip(ours, ref):
            torch.testing.assert_close(a.data, b.data, rtol=2e-6, atol=1e-7)
        assert all(p._version > v for p, v in zip(ours, versions))       # caches keyed on the version see the update
        opt.zero_grad(); topt.zero_grad()
    # the moments too
    for i in (0, 1, len(ours) - 1):
        st = topt.state[ref[i]]
        k = [id(p) for p in opt.params].index(id(ours[i]))
        for mine, theirs in ((opt._segment(opt.exp_avg, k), st["exp_avg"]), (opt._segment(opt.exp_avg_sq, k), st["exp_avg_sq"])):
            torch.testing.assert_close(mine, theirs, rtol=2e-6, atol=2e-7 * float(theirs.abs().max()))


def test_loss_scale_unscales_skips_and_grows():
    """GradScaler's rule on the device: scaled gradients give the same update as unscaled ones; a non-finite gradient skips the
    step and halves the scale; growth_interval good steps in a row double it."""
    from jetfire_int8training_b200.optim import ClipAdamW
    shapes = [(256, 128), (128,), (4100,)]
    ours, ref = _make(shapes, 5), _make(shapes, 5)
    opt = ClipAdamW([(ours, 0.1)], lr=1e-3, max_norm=1.0, loss_scale=1024.0, growth_interval=2)
    topt = torch.optim.AdamW(ref, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    gen = torch.Generator().manual_seed(6)
    scales = []
    for step in range(5):
        poison = step == 2
        scale = float(opt.state[0])
        for a, b in zip(ours, ref):
            gr = torch.randn(a.shape, generator=gen).to(DEV)
            a.grad = gr * scale
            b.grad = gr.clone()
        if poison:
            ours[1].grad[7] = float("inf")
        before = [p.detach().clone() for p in ours]
        out = opt.step()
        if poison:
            assert float(out[2]) == 1.0 and all(torch.equal(p.data, q) for p, q in zip(ours, before))     # nothing changed ...
            assert float(opt.state[0]) == scale * 0.5                                                      # ... but the scale
        else:
            assert float(out[2]) == 0.0
            tn = torch.nn.utils.clip_grad_norm_(ref, 1.0)
            topt.step()
            assert abs(float(out[0]) - float(tn)) <= 1e-5 * float(tn)
            for a, b in zip(ours, ref):
                torch.testing.assert_close(a.data, b.data, rtol=2e-6, atol=1e-7)
        scales.append(float(opt.state[0]))
    assert scales == [1024.0, 2048.0, 1024.0, 1024.0, 2048.0]
    assert opt.step_count == 4                                            # the skipped step does not count
    loss = torch.ones((), device=DEV, requires_grad=True)
    assert float(opt.scale_loss(loss)) == 2048.0


def test_parameters_become_views_of_one_buffer():
    from jetfire_int8training_b200.optim import ClipAdamW
    ps = _make([(8, 8), (4,)], 3)
    before = [p.detach().clone() for p in ps]
    opt = ClipAdamW([(ps, 0.0)], lr=1e-3)
    for p, b in zip(ps, before):
        assert torch.equal(p.data, b)
        lo, hi = opt.flat.data_ptr(), opt.flat.data_ptr() + opt.flat.numel() * 4
        assert lo <= p.data_ptr() < hi
    with pytest.raises(RuntimeError):
        opt.step()                       # no gradients yet
