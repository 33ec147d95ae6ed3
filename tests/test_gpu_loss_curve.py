"""GPU, end to end: the loss curve of a small GPT-2 trained on the CUDA operators must track the same model trained on the
reference's INT8 recipe restated in plain torch (tests/torch_recipe.py) -- same initial weights, same batches, same
optimiser; only the stochastic-rounding noise streams differ.  Tolerance: the mean loss over every 50-step window agrees
within 2 %, over the last 100 steps within 1 %."""
import contextlib
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu
DEV = "cuda"


@contextlib.contextmanager
def recipe_ops():
    """Run gpt2.QGPT on the torch restatement of the operators instead of the CUDA library."""
    import torch_recipe
    from jetfire_int8training_b200 import gpt2
    saved = gpt2.L, gpt2.NL, gpt2.lm_cross_entropy
    gpt2.L = gpt2.NL = torch_recipe
    gpt2.lm_cross_entropy = lambda logits, t: torch.nn.functional.cross_entropy(logits.float().view(-1, logits.size(-1)), t.view(-1))
    try:
        yield
    finally:
        gpt2.L, gpt2.NL, gpt2.lm_cross_entropy = saved


def synthetic_tokens(n_seq, T, vocab, seed):
    """A learnable stream: next token = (5 * current + 17 + small noise) mod vocab."""
    g = torch.Generator().manual_seed(seed)
    cur = torch.randint(0, vocab, (n_seq,), generator=g)
    cols = [cur]
    for _ in range(T):
        cur = (5 * cur + 17 + torch.randint(0, 3, (n_seq,), generator=g)) % vocab
        cols.append(cur)
    return torch.stack(cols, 1).to(DEV)


def train(model, data, steps, batch, use_recipe):
    opt = torch.optim.AdamW(model.parameters(), lr=2e-3, betas=(0.9, 0.95), weight_decay=0.0)
    losses = []
    ctx = recipe_ops() if use_recipe else contextlib.nullcontext()
    with ctx:
        for i in range(steps):
            rows = torch.arange(i * batch, (i + 1) * batch) % data.shape[0]
            ids = data[rows]
            loss = model(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())
            opt.zero_grad(set_to_none=True)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
            losses.append(float(loss.detach()))
    return torch.tensor(losses)


def test_loss_curve_tracks_the_reference_recipe():
    from jetfire_int8training_b200 import rng
    from jetfire_int8training_b200.gpt2 import GPTConfig, QGPT
    torch.manual_seed(0)
    rng.manual_seed(0)
    cfg = GPTConfig(block_size=64, vocab_size=512, n_layer=2, n_head=4, n_embd=128)
    ours = QGPT(cfg).to(DEV)
    theirs = copy.deepcopy(ours)
    data = synthetic_tokens(256, cfg.block_size, cfg.vocab_size, seed=1)
    steps, batch = 300, 8
    a = train(ours, data, steps, batch, use_recipe=False)
    torch.manual_seed(1)
    b = train(theirs, data, steps, batch, use_recipe=True)
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    assert a[-50:].mean() < 0.6 * a[:10].mean()                      # it learns
    print("window means ours / recipe:", [(round(float(a[w:w + 50].mean()), 4), round(float(b[w:w + 50].mean()), 4)) for w in range(0, steps, 50)])
    for w in range(0, steps, 50):
        ma, mb = float(a[w:w + 50].mean()), float(b[w:w + 50].mean())
        assert abs(ma - mb) <= 0.02 * mb, (w, ma, mb)
    ma, mb = float(a[-100:].mean()), float(b[-100:].mean())
    assert abs(ma - mb) <= 0.01 * mb, (ma, mb)
