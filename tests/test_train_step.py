"""CPU checks of the train-step harness (autoresearch_b200/train_step.py) on a tiny configuration, with
a plain-torch attention back end standing in for the library: the hand-written backward without
the reference's quirks equals autograd of an independently written forward; with the quirks it
differs exactly where the reference's backward is known to; the weight initialisation reproduces the
reference's generators; gradients are averaged over two gloo ranks."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import autoresearch_b200 as ab
from autoresearch_b200 import train_step as ts
from tests.torch_attention import TorchAttention, masked_attention, rope

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = ab.GPTConfig(sequence_len=24, vocab_size=50, n_layer=4, n_head=2, n_kv_head=2, n_embd=256, head_dim=128)


def tiny_weights(seed=0, dtype=torch.float64):
    w = ts.init_weights(CFG, "cpu", test_init=True)
    g = torch.Generator().manual_seed(seed)
    for k in w:                                   # break the symmetries of the reference's initial values
        if k.startswith("ve_gate") or k in ("resid_lambdas", "x0_lambdas"):
            w[k] = w[k] + 0.3 * torch.randn(w[k].shape, generator=g)
        if k == "lm_head":
            w[k] = w[k] * 300                      # logits large enough for the soft-cap to matter
    return {k: v.to(dtype) for k, v in w.items()}


def autograd_loss(w, ids, targets, cfg):
    """The model, written once more without reference to train_step's forward."""
    B, T = ids.shape
    H, D, C = cfg.n_head, cfg.head_dim, cfg.n_embd
    cos, sin = (torch.from_numpy(a).double() for a in ab.precompute_rope(T, D))

    def norm(x):
        return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)

    flat = ids.reshape(-1)
    x = norm(w["wte"][flat])
    x0 = x
    for i in range(cfg.n_layer):
        x = w["resid_lambdas"][i] * x + w["x0_lambdas"][i] * x0
        xn = norm(x)
        q, k, v = (xn @ w[f"{n}.{i}"].t() for n in ("c_q", "c_k", "c_v"))
        if cfg.has_ve(i):
            gate = 2 * torch.sigmoid(xn[:, :32] @ w[f"ve_gate.{i}"].t())
            v = (v.view(-1, H, D) + gate[..., None] * w[f"value_embeds.{i}"][flat].view(-1, H, D)).reshape(-1, C)
        q4, k4 = (norm(rope(t.view(B, T, H, D), cos, sin)) for t in (q, k))
        o = masked_attention(q4, k4, v.view(B, T, H, D), cfg.window_size(i)).reshape(-1, C)
        x = x + o @ w[f"c_proj.{i}"].t()
        x = x + torch.relu(norm(x) @ w[f"c_fc.{i}"].t()).pow(2) @ w[f"mlp_proj.{i}"].t()
    logits = 15 * torch.tanh(norm(x) @ w["lm_head"].t() / 15)
    return torch.nn.functional.cross_entropy(logits, targets.reshape(-1))


def run_step(w, ids, targets, quirks):
    step = ts.TrainStep(CFG, w, TorchAttention(CFG, ids.shape[1]), reference_quirks=quirks, compute_dtype=torch.float64,
                        master_dtype=torch.float64)           # fp64 throughout, for a tight comparison
    loss = step.step(ids, targets)
    return loss, step.grads


def test_exact_backward_matches_autograd():
    torch.manual_seed(1)
    ids = torch.randint(0, CFG.vocab_size, (2, CFG.sequence_len))
    targets = torch.randint(0, CFG.vocab_size, (2, CFG.sequence_len))
    w = tiny_weights()
    wa = {k: v.clone().requires_grad_(True) for k, v in w.items()}
    loss_a = autograd_loss(wa, ids, targets, CFG)
    loss_a.backward()
    loss, grads = run_step(w, ids, targets, quirks=False)
    assert abs(float(loss) - float(loss_a.detach())) < 1e-9
    for k in w:
        want = wa[k].grad
        err = (grads[k] - want).abs().max() / (want.abs().max() + 1e-30)
        assert err < 1e-7, (k, float(err))


def test_reference_quirks_change_only_what_they_should():
    torch.manual_seed(2)
    ids = torch.randint(0, CFG.vocab_size, (2, CFG.sequence_len))
    targets = torch.randint(0, CFG.vocab_size, (2, CFG.sequence_len))
    w = tiny_weights()
    loss_e, exact = run_step(w, ids, targets, quirks=False)
    loss_q, quirk = run_step(w, ids, targets, quirks=True)
    assert float(loss_e) == float(loss_q)                      # the forward is the same
    # the soft-cap factor is dropped first, so every gradient differs; all stay finite, of the same
    # sign structure, and the lm_head gradient differs by exactly that factor's effect
    for k in w:
        assert torch.isfinite(quirk[k]).all(), k
    assert (quirk["lm_head"] - exact["lm_head"]).abs().max() > 0
    cos = torch.nn.functional.cosine_similarity(quirk["lm_head"].reshape(1, -1), exact["lm_head"].reshape(1, -1))
    assert float(cos) > 0.9


def test_init_generators_restated():
    """fill_uniform / fill_normal against a scalar evaluation of the reference's formulas."""
    def scalar_uniform(seed, tid, low, high):
        m64 = (1 << 64) - 1
        st = (seed + tid * 6364136223846793005 + 1442695040888963407) & m64
        st ^= st >> 12; st ^= (st << 25) & m64; st ^= st >> 27
        return np.float32(low) + np.float32(st & 0xFFFFFF) / np.float32(0x1000000) * np.float32(high - low)
    got = ts.fill_uniform(44, -0.5, 0.5, 1000)
    for tid in (0, 1, 17, 999):
        assert got[tid] == scalar_uniform(44, tid, -0.5, 0.5)
    n = ts.fill_normal(42, 1.0, 200000)
    assert abs(float(n.mean())) < 0.01 and abs(float(n.std()) - 1.0) < 0.01
    w = ts.init_weights(CFG, "cpu")
    assert float(w["c_proj.0"].abs().max()) == 0.0 and float(w["resid_lambdas"][0]) == 1.0 and abs(float(w["x0_lambdas"][0]) - 0.1) < 1e-7
    assert set(k for k in w if k.startswith("value_embeds")) == {"value_embeds.1", "value_embeds.3"}   # has_ve: i % 2 == (L-1) % 2


WORKER = r'''
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, %r)
import autoresearch_b200 as ab
from autoresearch_b200 import train_step as ts
from tests.torch_attention import TorchAttention
from tests.test_train_step import CFG, tiny_weights
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(5)
ids = torch.randint(0, CFG.vocab_size, (world, 2, CFG.sequence_len))
tg = torch.randint(0, CFG.vocab_size, (world, 2, CFG.sequence_len))
w = tiny_weights(dtype=torch.float32)
def grads_of(r, pg):
    st = ts.TrainStep(CFG, w, TorchAttention(CFG, CFG.sequence_len, torch.float32), reference_quirks=True,
                      compute_dtype=torch.float32, process_group=pg)
    st.step(ids[r], tg[r])
    return st.grads
mine = grads_of(rank, True)                     # gradients averaged over the ranks, bucket by bucket
local = [grads_of(r, None) for r in range(world)]
for k in w:
    want = sum(g[k] for g in local) / world
    assert torch.allclose(mine[k], want, rtol=1e-5, atol=1e-7), k
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_rank_gloo_gradient_allreduce(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29741", str(script)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2
