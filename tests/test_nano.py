"""The single-file readable implementation runs and behaves: faithful after training, unmasked = target."""
import itertools

import torch
from torch import nn

from param_decomp_b200 import nano


class TinyLM(nn.Module):
    def __init__(self, vocab=37, d=16):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.fc1, self.fc2 = nn.Linear(d, 32), nn.Linear(32, d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, tokens):
        x = self.emb(tokens)
        x = x + self.fc2(torch.relu(self.fc1(x)))
        return self.head(x)


def test_nano_decompose_and_evaluate():
    torch.manual_seed(0)
    model = TinyLM()
    g = torch.Generator().manual_seed(1)
    data = (torch.randint(0, 37, (8, 12), generator=g) for _ in itertools.count())
    cfg = nano.NanoConfig(n_components=24, ci_hidden=16, steps=60, faithfulness_warmup_steps=40, lr=3e-3, log_every=20)
    tokens = torch.randint(0, 37, (8, 12), generator=g)
    before = model(tokens)
    comps, ci_net = nano.decompose(model, ["fc1", "fc2"], data, cfg)
    assert set(comps) == {"fc1", "fc2"} and cfg.history[-1]["step"] == 59
    assert cfg.history[-1]["faith"] < cfg.history[0]["faith"]
    assert torch.allclose(model(tokens), before, atol=1e-6)  # masks off: the wrapped model IS the target
    ev = nano.evaluate(model, comps, ci_net, tokens)
    assert ev["kl/unmasked"] < 1e-6 and ev["kl/zero_masked"] > ev["kl/unmasked"]
    assert all(v == v for v in ev.values())


def test_lower_leaky_gradient_rule():
    x = torch.tensor([-1.0, -1.0, 0.5, 2.0], requires_grad=True)
    nano.lower_leaky(x, 0.01).backward(torch.tensor([1.0, -1.0, 3.0, 5.0]))
    assert torch.allclose(x.grad, torch.tensor([0.0, -0.01, 3.0, 0.0]))
