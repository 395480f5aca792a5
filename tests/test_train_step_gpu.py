"""GPU test of the train-step harness with the library's attention back end (and, with
projections="library", the library's projection GEMMs in place of torch's): on a small model the
loss and the gradients agree with the same step run on the CPU in fp64 with the plain-torch attention
stand-in, to the accuracy bf16 matmul operands allow."""
import pytest
import torch

import autoresearch_b200 as ab
from autoresearch_b200 import train_step as ts
from tests.torch_attention import TorchAttention

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("projections", ["torch", "library"])
@pytest.mark.parametrize("quirks", [True, False])
def test_step_matches_cpu_fp64(cuda_device, quirks, projections):
    cfg = ab.GPTConfig(sequence_len=384, vocab_size=512, n_layer=4, n_head=2, n_kv_head=2, n_embd=256, head_dim=128)
    B, T = 2, cfg.sequence_len
    torch.manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (B, T))
    targets = torch.randint(0, cfg.vocab_size, (B, T))
    w = ts.init_weights(cfg, "cpu", test_init=True)
    g = torch.Generator().manual_seed(1)
    for k in list(w):
        if k.startswith("ve_gate"):
            w[k] = w[k] + 0.3 * torch.randn(w[k].shape, generator=g)
        # The reference's generator gives c_q, c_k, c_v of a layer nearly the same values (consecutive
        # seeds), which makes every query attend to itself alone; in that corner dQ, dK are a tiny
        # residual of cancelling terms and no bf16 kernel can be compared element by element.  The
        # comparison uses independent matrices of the same scale.
        if k.startswith(("c_q", "c_k", "c_v")):
            w[k] = (torch.rand(w[k].shape, generator=g) * 2 - 1) * float(w[k].abs().max())
    ref = ts.TrainStep(cfg, {k: v.double() for k, v in w.items()}, TorchAttention(cfg, T), reference_quirks=quirks,
                       compute_dtype=torch.float64, master_dtype=torch.float64)
    loss_ref = ref.step(ids, targets)
    wd = {k: v.cuda() for k, v in w.items()}
    dev = ts.TrainStep(cfg, wd, ts.LibraryAttention(cfg, T, "cuda"), reference_quirks=quirks,
                       projections=projections)
    loss_dev = dev.step(ids.cuda(), targets.cuda())
    ab.check_device_status()
    assert abs(float(loss_dev) - float(loss_ref)) < 2e-3 * float(loss_ref)
    for k in w:
        a, b = dev.grads[k].double().cpu().reshape(-1), ref.grads[k].reshape(-1)
        cos = torch.nn.functional.cosine_similarity(a, b, dim=0)
        rel = (a - b).norm() / (b.norm() + 1e-30)
        assert float(cos) > 0.995 and float(rel) < 0.1, (k, float(cos), float(rel))
    assert dev.attention.attention_ms() > 0
