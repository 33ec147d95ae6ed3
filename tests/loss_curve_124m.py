"""GPU script (not collected by pytest): the loss curve of GPT-2 124M trained on the CUDA operators next to the same model trained
on the reference's INT8 recipe restated in plain torch (tests/torch_recipe.py, pinned to the golden vectors of the reference's own
kernels by tests/test_recipe_golden.py) -- same initial weights, same batches, same optimiser; only the stochastic-rounding noise
streams differ.

    python tests/loss_curve_124m.py [--steps 2000] [--micro-batch 12] [--layers 12] [--stream learnable|uniform] [--seed-variance | --compare-optimizers]

GPT-2 124M: 12 layers, 12 heads, d = 768, context 1024, vocabulary 50304, AdamW lr 6e-4 (100 warm-up steps), betas (0.9, 0.95),
weight decay 0.1, gradient clipping 1.0, loss scaling as the reference's GradScaler (init 2^24; the fp16 gradients that cross the
attention underflow without it).  Every forward pass quantises the current weights.  Token stream: seeded synthetic ids.  `uniform` draws them uniformly (nothing can be
learnt: the curve stays at ln 50304); `learnable` (default) makes the next token (5 t + 17 + {0,1,2}) mod 50304, so the loss
falls and a mismatch between the two implementations would show.  Prints one JSON line with the mean loss of every 100-step
window for both runs and the largest relative gap between them.  --seed-variance runs the CUDA operators twice instead, with
two different stochastic-rounding seeds and everything else equal: the gap between those two curves is the run-to-run spread of
ONE implementation, the yardstick for the gap between two implementations (it is largest where the loss falls fastest).
"""
import argparse
import contextlib
import copy
import json
import os
import sys
import time

import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
DEV = "cuda"


@contextlib.contextmanager
def recipe_ops():
    """Run gpt2.QGPT on the torch restatement of the operators (and torch's own cross-entropy) instead of the CUDA library."""
    import torch_recipe
    from jetfire_int8training_b200 import gpt2
    saved = gpt2.L, gpt2.NL, gpt2.lm_cross_entropy
    gpt2.L = gpt2.NL = torch_recipe
    gpt2.lm_cross_entropy = lambda logits, t: F.cross_entropy(logits.float().view(-1, logits.size(-1)), t.view(-1))
    try:
        yield
    finally:
        gpt2.L, gpt2.NL, gpt2.lm_cross_entropy = saved


def batches(steps, mb, T, vocab, stream, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    for _ in range(steps):
        if stream == "uniform":
            ids = torch.randint(0, vocab, (mb, T + 1), generator=g, device=DEV)
        else:
            cur = torch.randint(0, vocab, (mb,), generator=g, device=DEV)
            noise = torch.randint(0, 3, (mb, T), generator=g, device=DEV)
            cols = [cur]
            for k in range(T):
                cur = (5 * cur + 17 + noise[:, k]) % vocab
                cols.append(cur)
            ids = torch.stack(cols, 1)
        yield ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def train(model, args, use_recipe, fused_optimizer=False):
    """Loss scaling as in the reference's loop (INT8_GPT2/train.py:216-217, 320-327): GradScaler(init_scale=2**24), unscale, clip
    to norm 1.0, step, update.  Returns (losses, number of steps the scaler skipped)."""
    decay = [p for p in model.parameters() if p.dim() >= 2]
    nodecay = [p for p in model.parameters() if p.dim() < 2]
    if fused_optimizer:
        from jetfire_int8training_b200.optim import ClipAdamW
        opt = ClipAdamW([(decay, 0.1), (nodecay, 0.0)], lr=6e-4, betas=(0.9, 0.95), max_norm=1.0, loss_scale=2.0 ** 24)
        scaler = None
    else:
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}], lr=6e-4,
                                betas=(0.9, 0.95), fused=True)
        scaler = torch.amp.GradScaler("cuda", init_scale=2.0 ** 24)
    losses = []
    ctx = recipe_ops() if use_recipe else contextlib.nullcontext()
    t0 = time.time()
    with ctx:
        for i, (x, y) in enumerate(batches(args.steps, args.micro_batch, model.cfg.block_size, model.cfg.vocab_size, args.stream, 1234)):
            lr = 6e-4 * min(1.0, (i + 1) / 100.0)
            if fused_optimizer:
                opt.lr = lr
            else:
                for grp in opt.param_groups:
                    grp["lr"] = lr
            loss = model(x, y)
            opt.zero_grad(set_to_none=True)
            if fused_optimizer:
                opt.scale_loss(loss).backward()
                opt.step()              # unscales, clips to norm 1.0, steps and updates the scale itself
            else:
                scaler.scale(loss).backward()
                scaler.unscale_(opt)
                torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
                scaler.step(opt)
                scaler.update()
            losses.append(loss.detach())
            if (i + 1) % 100 == 0:
                sc = float(opt.state[0]) if fused_optimizer else scaler.get_scale()
                print(f"{'recipe' if use_recipe else 'cuda'} step {i + 1}: loss {float(losses[-1]):.4f}  loss scale {sc:g}  ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    return torch.stack(losses).float().cpu()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--micro-batch", type=int, default=12)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--stream", default="learnable", choices=["learnable", "uniform"])
    ap.add_argument("--seed-variance", action="store_true")
    ap.add_argument("--compare-optimizers", action="store_true",
                    help="CUDA operators twice, same stochastic-rounding seed: optim.ClipAdamW against clip_grad_norm_ + torch AdamW")
    args = ap.parse_args()
    from jetfire_int8training_b200 import rng
    from jetfire_int8training_b200.gpt2 import GPTConfig, QGPT
    torch.manual_seed(0)
    rng.manual_seed(0)
    cfg = GPTConfig(n_layer=args.layers)
    ours = QGPT(cfg).to(DEV)
    theirs = copy.deepcopy(ours)
    a = train(ours, args, use_recipe=False, fused_optimizer=args.compare_optimizers)
    del ours
    torch.cuda.empty_cache()
    torch.manual_seed(1)
    if args.compare_optimizers:
        rng.manual_seed(0)                           # the same stochastic-rounding stream: only the optimiser step differs
        b = train(theirs, args, use_recipe=False)
    elif args.seed_variance:
        rng.manual_seed(12345)                       # a different stochastic-rounding stream, same weights and batches
        b = train(theirs, args, use_recipe=False)
    else:
        b = train(theirs, args, use_recipe=True)
    w = 100
    wins = [(round(float(a[i:i + w].mean()), 4), round(float(b[i:i + w].mean()), 4)) for i in range(0, args.steps - w + 1, w)]
    gap = max(abs(x - y) / y for x, y in wins)
    print(json.dumps({"model": f"GPT-2 124M shape, {args.layers} layers", "steps": args.steps, "micro_batch": args.micro_batch, "stream": args.stream,
                      "window": w, "compared": ("cuda with optim.ClipAdamW vs cuda with clip_grad_norm_ + torch AdamW" if args.compare_optimizers else
                                   "cuda (SR seed 0) vs cuda (SR seed 12345)" if args.seed_variance else "cuda vs recipe"),
                      "window_means_cuda_vs_recipe": wins, "max_relative_gap_of_window_means": gap,
                      "first_loss": [float(a[0]), float(b[0])], "last_window": wins[-1], "finite": bool(torch.isfinite(a).all() and torch.isfinite(b).all())}))


if __name__ == "__main__":
    main()
