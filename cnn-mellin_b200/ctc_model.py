"""The CNN-CTC acoustic-model training step the Mellin layers are benchmarked in.

A synthetic stand-in for the reference's training loop
(``running.py:240,280-291``: CTC loss with the blank as last class, backward,
optimizer step) around the reference's conv block (``models.py:424-434``:
conv -> nonlinearity -> dropout, inputs multiplied by the length mask): ten
Mellin x linear layers over (3, 41 bins, T frames) features, two hidden
fully-connected layers of width 1024 on every frame, a 62-way output (61
phones + blank), ``log_softmax``, ``CTCLoss(blank=61, zero_infinity=True)``,
Adam with learning rate 1e-4, FP32 throughout.

Only the convolutional layers are this package's kernels; the per-frame
matrix products, the loss and the optimizer are stock PyTorch, as they are in
the reference.  Data is synthetic: N(0, 1) features of ragged length, random
label sequences.
"""
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

import mconv

BINS = 41
CLASSES = 62  # 61 phones + blank (the last index, as running.py:240)
CHANNELS = (3, 128, 128, 128, 128, 128, 256, 256, 256, 256, 256)
KERNEL = (6, 3)


class _PackFrames(torch.autograd.Function):
    """(N, K, T) padded features -> (K, sum of lengths): the frames inside each utterance, utterance by utterance."""

    @staticmethod
    def forward(ctx, x, lengths):
        ctx.lengths, ctx.shape = lengths, x.shape
        return torch.cat([x[i, :, :n] for i, n in enumerate(lengths)], dim=1)

    @staticmethod
    def backward(ctx, grad):
        gx = grad.new_zeros(ctx.shape)
        o = 0
        for i, n in enumerate(ctx.lengths):
            gx[i, :, :n] = grad[:, o:o + n]
            o += n
        return gx, None


class _UnpackFrames(torch.autograd.Function):
    """(C, sum of lengths) -> (T, N, C) padded with zeros: the layout the CTC loss reads."""

    @staticmethod
    def forward(ctx, packed, lengths, t):
        ctx.lengths = lengths
        out = packed.new_zeros((t, len(lengths), packed.shape[0]))
        o = 0
        for i, n in enumerate(lengths):
            out[:n, i] = packed[:, o:o + n].t()
            o += n
        return out

    @staticmethod
    def backward(ctx, grad):
        return torch.cat([grad[:n, i].t() for i, n in enumerate(ctx.lengths)], dim=1), None, None


class MellinCTCNet(torch.nn.Module):
    def __init__(self, channels: Sequence[int] = CHANNELS, kernel: Tuple[int, int] = KERNEL, bins: int = BINS,
                 hidden: int = 1024, classes: int = CLASSES, dropout: float = 0.05, fused_dropout: bool = True):
        super().__init__()
        valid = mconv.mcorr_valid_size(kernel[0], bins)
        same = (bins - valid, 1)  # same-size output on both axes (time padding 1)
        self.convs = torch.nn.ModuleList(
            mconv.MCorrLCorr(ci, co, kernel, s=1, d=(1, 1), p=(0, 1), r=same)
            for ci, co in zip(channels[:-1], channels[1:]))
        for conv in self.convs:
            torch.nn.init.kaiming_normal_(conv.weight)
            torch.nn.init.zeros_(conv.bias)
        self.dropout = dropout
        self.fused_dropout = fused_dropout  # False: torch's dropout as a separate pass (for comparison)
        self.fc1 = torch.nn.Linear(channels[-1] * bins, hidden)
        self.fc2 = torch.nn.Linear(hidden, hidden)
        self.out = torch.nn.Linear(hidden, classes)

    def forward(self, x: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        """x: (N, 3, bins, T) zero beyond lens[n] frames; lens: int32 (N,).  Returns (T, N, classes) log-probabilities."""
        for conv in self.convs:
            # dropout(relu(conv(x)) * mask): the reference's conv -> nonlinearity -> dropout block in one kernel
            if self.fused_dropout:
                x = mconv.mcorrlcorr_masked(x, conv.weight, conv.bias, lens, True, conv.s, conv.d, conv.p, conv.r,
                                            dropout_p=self.dropout, training=self.training)
            else:
                x = mconv.mcorrlcorr_masked(x, conv.weight, conv.bias, lens, True, conv.s, conv.d, conv.p, conv.r)
                x = F.dropout(x, self.dropout, self.training)
        n, c, b, t = x.shape
        # Only the frames inside the utterances go through the per-frame layers (the reference packs its frames the
        # same way before its recurrent layers, models.py:407-411): features (c * bins, frames) gathered utterance by
        # utterance, so that W @ h needs no transposition and the ~37 % of padding costs nothing.
        lengths = [min(int(v), t) for v in lens.tolist()]
        h = _PackFrames.apply(x.reshape(n, c * b, t), lengths)                        # (features, valid frames)
        h = F.relu(torch.addmm(self.fc1.bias[:, None], self.fc1.weight, h))
        h = F.relu(torch.addmm(self.fc2.bias[:, None], self.fc2.weight, h))
        logits = torch.addmm(self.out.bias[:, None], self.out.weight, h)              # (classes, valid frames)
        # back to the padded (T, N, classes) layout the loss expects; frames past an utterance's end are never read
        return _UnpackFrames.apply(F.log_softmax(logits, dim=0), lengths, t)


def synthetic_lengths(count: int, seed: int, lo: int = 200, hi: int = 800) -> List[int]:
    """Frame counts T ~ Uniform{lo..hi} of `count` utterances (same list on every rank for the same seed)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi + 1, (count,), generator=gen).tolist()


def synthetic_batch(lengths: Sequence[int], seed: int, device, bins: int = BINS, pad_to_multiple: int = 4):
    """Features zero-padded to the longest utterance (rounded up to a multiple of 4 frames, the kernels' 16-byte
    row granularity), lengths, and random label sequences of length ~ U{20..80} over the 61 phones."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    n = len(lengths)
    t_max = (max(lengths) + pad_to_multiple - 1) // pad_to_multiple * pad_to_multiple
    x = torch.randn((n, 3, bins, t_max), generator=gen)
    lens = torch.tensor(lengths, dtype=torch.int32)
    x *= (torch.arange(t_max)[None, :] < lens[:, None])[:, None, None, :]
    target_lengths = torch.randint(20, 81, (n,), generator=gen)
    targets = torch.randint(0, CLASSES - 1, (int(target_lengths.sum()),), generator=gen)
    return x.to(device), lens.to(device), targets.to(device), target_lengths.to(device)


def ctc_loss(log_probs: torch.Tensor, lens: torch.Tensor, targets: torch.Tensor, target_lengths: torch.Tensor):
    return F.ctc_loss(log_probs, targets, lens.long(), target_lengths, blank=CLASSES - 1, zero_infinity=True)


class TrainStep:
    """One data-parallel training step: forward, CTC loss, backward with the
    gradient buckets all-reduced while backward still runs, Adam update."""

    def __init__(self, model: MellinCTCNet, lr: float = 1e-4, reducer=None):
        self.model = model
        self.reducer = reducer
        self.optimizer = torch.optim.Adam(model.parameters(), lr=lr, fused=next(model.parameters()).is_cuda)

    def __call__(self, x, lens, targets, target_lengths) -> torch.Tensor:
        self.model.train()
        if self.reducer is not None:
            self.reducer.begin_step()
        else:
            self.optimizer.zero_grad(set_to_none=False)
        loss = ctc_loss(self.model(x, lens), lens, targets, target_lengths)
        loss.backward()
        if self.reducer is not None:
            self.reducer.finish_step()
        self.optimizer.step()
        return loss.detach()
