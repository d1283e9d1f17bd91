"""The transformer CI functions on the sm_100a path: their linears on the tcgen05 GEMM, their attention on the
flash kernel (shapes outside the kernel's native range are padded to it), the routed expert bank as grouped
products - each against the plain fp32 PyTorch evaluation of the same module."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("T,hd,causal,segments", [(200, 34, False, True), (96, 64, True, False), (256, 40, True, True)])
def test_flash_attention_pads_odd_shapes(T, hd, causal, segments):
    from param_decomp_b200.models import ports
    from param_decomp_b200.ops import native

    torch.manual_seed(0)
    B, H, Hkv = 2, 4, 2
    q = torch.randn(B, T, H, hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    seg = None
    if segments:
        seg = (torch.arange(T, device="cuda")[None] >= torch.tensor([[T // 3], [T // 2]], device="cuda")).int()
    out = ports.sdpa(q, k, v, causal, seg, "flash")
    g = torch.randn_like(out)
    out.backward(g)
    qe, ke, ve = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = ports.sdpa_reference(qe, ke, ve, causal, seg)
    ref.backward(g.float())
    native.check_status()
    assert out.shape == ref.shape
    assert rel(out, ref) < 2e-2
    assert rel(q.grad, qe.grad) < 4e-2 and rel(k.grad, ke.grad) < 4e-2 and rel(v.grad, ve.grad) < 4e-2


def test_flash_attention_refuses_what_it_cannot_do():
    from param_decomp_b200.models import ports

    q = torch.randn(1, 128, 2, 160, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        ports.sdpa(q, q, q, True, None, "flash")


def test_global_transformer_ci_fused_matches_eager():
    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.core.ci_fn.transformer import FusedLinear
    from param_decomp_b200.experiments.lm.build import build_lm_run
    from param_decomp_b200.ops import native

    dev = torch.device("cuda", 0)
    outs = {}
    for backend in ("eager_torch", "fused_sm100"):
        c = copy.deepcopy(ge.SMOKE_CONFIG)
        c["runtime"]["backend"] = backend
        c["decomposition"]["ci"] = {
            "type": "global_transformer", "d_model": 136, "n_blocks": 2,
            "attention": {"kind": "mha", "n_heads": 4, "implementation": "flash", "mask": "bidirectional"},  # head_dim 34
            "ffn": {"kind": "swiglu", "hidden": 192}, "input_tap": {"kind": "residual_boundaries", "offsets": [0, 1, 2]}}
        cfg = LMExperimentConfig.model_validate(c)
        run = build_lm_run(cfg, None, dev)
        ci_fn = run.ci_fn.to(dev)
        fused = [m for m in ci_fn.modules() if isinstance(m, FusedLinear) and m.fused]
        assert bool(fused) == (backend == "fused_sm100")
        with torch.no_grad():
            clean = run.model.clean_forward(run.sample_train(0))
        pre = ci_fn(clean.taps, aux=clean.aux, components=None, segment_ids=None, positions=None)
        loss = sum((p.float() ** 2).mean() for p in pre.values())
        loss.backward()
        outs[backend] = ({k: v.detach().float() for k, v in pre.items()},
                         {n: p.grad.detach().float() for n, p in ci_fn.named_parameters() if p.grad is not None})
    native.check_status()
    pe, ge_ = outs["eager_torch"]
    pf, gf = outs["fused_sm100"]
    for k in pe:
        assert rel(pf[k], pe[k]) < 4e-2, (k, rel(pf[k], pe[k]))
    big = [n for n in ge_ if ge_[n].dim() == 2]
    assert big and all(rel(gf[n], ge_[n]) < 8e-2 for n in big), {n: rel(gf[n], ge_[n]) for n in big}


def test_routed_linear_grouped_matches_per_expert_loop():
    from param_decomp_b200.core.ci_fn.transformer import routed_linear
    from param_decomp_b200.core.components import BlockSelection
    from param_decomp_b200.ops import native

    torch.manual_seed(1)
    N, k, E, d, h = 300, 2, 6, 64, 48
    idx = torch.stack([torch.randperm(E - 1, device="cuda")[:k] for _ in range(N)])  # expert E-1 gets no job
    sel = BlockSelection(idx.view(1, N, k), torch.rand(1, N, k, device="cuda"))
    x = torch.randn(N, d, device="cuda")
    W = (torch.randn(E, d, h, device="cuda") / d**0.5).requires_grad_(True)
    out = routed_linear(x, W, sel, per_job=False, fused=True)
    out.float().pow(2).sum().backward()
    We = W.detach().clone().requires_grad_(True)
    ref = routed_linear(x.to(torch.bfloat16).float(), We, sel, per_job=False, fused=False)
    ref.pow(2).sum().backward()
    native.check_status()
    assert rel(out, ref) < 2e-2 and rel(W.grad, We.grad) < 4e-2
    assert float(W.grad[E - 1].abs().sum()) == 0.0


def test_streamed_vocab_kl_matches_materialised_and_bounds_memory():
    """`output_edge: streamed` on the fused backend: same loss and hidden-state gradient as the materialised
    form, and no `[positions, vocab]` tensor - peak extra memory stays near 3 x chunk x vocab bf16."""
    from param_decomp_b200.ops import native, vocab_kl

    torch.manual_seed(0)
    n, d, V, rows = 16384, 256, 50272, 512
    head = (torch.randn(V, d, device="cuda") / d**0.5).to(torch.bfloat16)
    hc = torch.randn(n, d, device="cuda", dtype=torch.bfloat16)
    hm = (hc.float() + 0.3 * torch.randn(n, d, device="cuda")).to(torch.bfloat16)
    a = hm.clone().requires_grad_(True)
    la = vocab_kl.kl_from_hidden(vocab_kl.padded_logits(hc, head), a, head)
    (la * 3.0).backward()
    del la
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    b = hm.clone().requires_grad_(True)
    lb = vocab_kl.kl_from_hidden_streamed(hc, b, head, rows)
    (lb * 3.0).backward()
    torch.cuda.synchronize()
    native.check_status()
    peak = torch.cuda.max_memory_allocated() - base
    one_full = n * V * 2
    assert peak < 3.5 * rows * V * 2 + 16 * n * d, (peak, rows * V * 2)
    assert peak < 0.15 * one_full  # far below even ONE materialised logits tensor
    la2 = vocab_kl.kl_from_hidden(vocab_kl.padded_logits(hc, head), hm, head)
    assert float(lb) == pytest.approx(float(la2), rel=2e-3)
    assert rel(b.grad, a.grad) < 2e-3
