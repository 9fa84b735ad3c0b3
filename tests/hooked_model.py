"""A small engine-style model whose parameters carry ``weight_loader`` hooks, the
convention vLLM uses and the one the reference's geometry capture stamps
(refit/reshard/geometry.py:206-250).  It is shared by the fixture generator,
which runs the REFERENCE's capture on it, and by the test that runs this
repository's capture on it, so both see the same loaders."""

import torch

TP, RANK = 4, 1
HIDDEN, QH, KVH, HD, INTER, VOCAB, EXPERTS = 32, 8, 4, 4, 48, 40, 3


def _column(param, w, shard_id=None):
    rows = param.shape[0]
    param.data.copy_(w.narrow(0, RANK * rows, rows))


def _row(param, w):
    cols = param.shape[1]
    param.data.copy_(w.narrow(1, RANK * cols, cols))


def _qkv(param, w, shard_id):
    per = {"q": QH * HD // TP, "k": KVH * HD // TP, "v": KVH * HD // TP}
    at = {"q": 0, "k": per["q"], "v": per["q"] + per["k"]}[shard_id]
    param.data.narrow(0, at, per[shard_id]).copy_(w.narrow(0, RANK * per[shard_id], per[shard_id]))


def _gate_up(param, w, shard_id):
    half = INTER // TP
    param.data[shard_id * half:(shard_id + 1) * half].copy_(w[RANK * half:(RANK + 1) * half])


def _pre_merged(param, w):
    # checkpoint stores [gate; up] already concatenated: take this rank's block of each half
    half = INTER // TP
    gate, up = w.chunk(2, dim=0)
    param.data[:half].copy_(gate.narrow(0, RANK * half, half))
    param.data[half:].copy_(up.narrow(0, RANK * half, half))


def _transposed(param, w):
    # stored (in, out); the parameter is (out / TP, in)
    rows = param.shape[0]
    param.data.copy_(w.t().narrow(0, RANK * rows, rows))


def _expert(param, w, expert_id):
    # per-expert checkpoint tensor (inter, hidden) into the stacked parameter
    half = INTER // TP
    param.data[expert_id].copy_(w.narrow(0, RANK * half, half))


def _vocab(param, w):
    rows = param.shape[0]
    lo = RANK * rows
    n = max(0, min(rows, w.shape[0] - lo))
    param.data[:n].copy_(w.narrow(0, lo, n))
    param.data[n:].fill_(0)


class HookedModel(torch.nn.Module):
    def __init__(self):
        super().__init__()
        P = torch.nn.Parameter

        def make(shape, loader):
            p = P(torch.zeros(shape))
            p.weight_loader = loader
            return p

        self.qkv = make(((QH + 2 * KVH) * HD // TP, HIDDEN), _qkv)
        self.o = make((HIDDEN, QH * HD // TP), _row)
        self.gate_up = make((2 * INTER // TP, HIDDEN), _gate_up)
        self.merged = make((2 * INTER // TP, HIDDEN), _pre_merged)
        self.down = make((HIDDEN, INTER // TP), _row)
        self.proj_t = make((HIDDEN // TP, HIDDEN), _transposed)
        self.experts = make((EXPERTS, INTER // TP, HIDDEN), _expert)
        self.embed = make((12, HIDDEN), _vocab)              # 40 rows padded to 48 = 4 x 12
        self.norm = P(torch.zeros(HIDDEN))                   # no hook: the default loader

    def load_weights(self, weights):
        params = dict(self.named_parameters())
        for name, w in weights:
            if name in ("q", "k", "v"):
                params["qkv"].weight_loader(params["qkv"], w, name)
            elif name in ("gate", "up"):
                params["gate_up"].weight_loader(params["gate_up"], w, 0 if name == "gate" else 1)
            elif name.startswith("expert."):
                params["experts"].weight_loader(params["experts"], w, int(name.split(".")[1]))
            else:
                p = params[name]
                loader = getattr(p, "weight_loader", default_weight_loader)
                loader(p, w)


def default_weight_loader(param, w):
    param.data.copy_(w)


def manifest():
    out = [("q", (QH * HD, HIDDEN)), ("k", (KVH * HD, HIDDEN)), ("v", (KVH * HD, HIDDEN)),
           ("o", (HIDDEN, QH * HD)), ("gate", (INTER, HIDDEN)), ("up", (INTER, HIDDEN)),
           ("merged", (2 * INTER, HIDDEN)), ("down", (HIDDEN, INTER)), ("proj_t", (HIDDEN, HIDDEN)),
           ("embed", (VOCAB, HIDDEN)), ("norm", (HIDDEN,))]
    out += [(f"expert.{e}", (INTER, HIDDEN)) for e in range(EXPERTS)]
    return [(n, torch.float32, s) for n, s in out]
