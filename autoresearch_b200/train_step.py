"""Forward + backward of the reference's small GPT around the attention library (BASELINE config 3).

A restatement, in PyTorch tensor operations, of the reference trainer's ``forward`` and ``backward``
(model.mojo:576-772, 819-1037) with the attention path - RoPE, per-head RMSNorm of q and k, flash
attention and its backward - handed to libarattn.so.  Everything else (embedding, RMSNorm, the
linear layers, squared-ReLU MLP, value embeddings with their gate, learned residual scalars, logit
soft-cap, cross-entropy) is plain torch: those kernels of the reference are outside the path this
package replaces, and here they only provide the realistic surroundings in which the attention
share of a training step is measured.

The model (config.mojo:9-55; train.py's GPT as the reference restates it):
    x = norm(wte[ids]); x0 = x
    per layer i:  x = resid_lambdas[i] * x + x0_lambdas[i] * x0
                  xn = norm(x); q, k, v = xn Wq^T, xn Wk^T, xn Wv^T
                  layers with a value embedding: v += 2 sigmoid(xn[:, :32] Wg^T) * value_embeds[ids]
                  q, k = norm_per_head(rope(q)), norm_per_head(rope(k))
                  x += attention(q, k, v, window_size(i)) Wproj^T
                  x += relu(norm(x) Wfc^T)^2 Wmlp^T
    logits = 15 tanh(norm(x) Wlm^T / 15);  loss = mean cross-entropy

``reference_quirks`` chooses between two backward passes.  False: the exact gradient of the forward
above (what autograd gives; checked against autograd in tests/test_train_step.py).  True: the
backward as the reference's ``backward`` computes it, which departs from the exact gradient in
these places (file:line in the reference):
  * the soft-cap's chain-rule factor 1 - tanh^2 is not applied (ops.mojo:854-864, model.mojo:847-855);
  * the per-head RMSNorm of q, k and the RMSNorm of the embedding pass gradients straight through
    (model.mojo:937, 1028-1031);
  * the MLP pre-norm backward is evaluated at the layer's pre-attention x (model.mojo:892-896);
  * the gradient of resid_lambdas is reduced against the layer's input after the scaled add instead of
    before it (model.mojo:1003-1007), and the gradient into x0 is overwritten per layer and never
    reaches the embedding (model.mojo:1014-1026).
The reference's matmul kernels write only a quarter of each output tile (ops.mojo:134-143) and its
c_proj backward reads and writes one buffer from many blocks (model.mojo:906); neither is a
numerical convention that could be followed, so both modes compute Y = X W^T and its gradients.

Data parallelism: every rank runs the same step on its own batch; ``allreduce_grads`` sums the
gradients over the ranks in per-layer buckets with NCCL (torch.distributed), launched as each
layer's backward finishes so that the transfers overlap the rest of the backward pass.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from .config import GPTConfig, precompute_rope

MLP_EXPANSION = 4        # config.mojo:63
VE_GATE_CHANNELS = 32    # config.mojo:64
SOFTCAP = 15.0           # config.mojo:86
NORM_EPS = 1e-5          # ops.mojo:97


# --------------------------------------------------------------------------------------------
# weights
# --------------------------------------------------------------------------------------------
def _xorshift(state: np.ndarray) -> np.ndarray:
    state = state ^ (state >> np.uint64(12))
    state = state ^ (state << np.uint64(25))
    state = state ^ (state >> np.uint64(27))
    return state


_MUL, _INC = np.uint64(6364136223846793005), np.uint64(1442695040888963407)


def fill_uniform(seed: int, low: float, high: float, size: int) -> np.ndarray:
    """model.mojo:121-137 (fill_uniform_kernel): one xorshift draw per element, 24 bits."""
    with np.errstate(over="ignore"):
        tid = np.arange(size, dtype=np.uint64)
        state = _xorshift(np.uint64(seed) + tid * _MUL + _INC)
    u = (state & np.uint64(0xFFFFFF)).astype(np.float32) / np.float32(0x1000000)
    return (np.float32(low) + u * np.float32(high - low)).astype(np.float32)


def fill_normal(seed: int, std: float, size: int) -> np.ndarray:
    """model.mojo:86-118 (fill_normal_kernel): two xorshift draws and a Box-Muller transform."""
    with np.errstate(over="ignore"):
        tid = np.arange(size, dtype=np.uint64)
        state = _xorshift(np.uint64(seed) + tid * _MUL + _INC)
        u1 = (state & np.uint64(0xFFFFFF)).astype(np.float32) / np.float32(0x1000000) + np.float32(1e-10)
        state = _xorshift(state * _MUL + _INC)
    u2 = (state & np.uint64(0xFFFFFF)).astype(np.float32) / np.float32(0x1000000)
    z = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(2.0 * math.pi) * u2)
    return (z * np.float32(std)).astype(np.float32)


def init_weights(cfg: GPTConfig, device, test_init: bool = False) -> Dict[str, torch.Tensor]:
    """The reference's initial weights (model.mojo:337-427), seeds 42, 43, ... in its order.

    Note what the generator does with consecutive seeds: only the lowest bit of its 24-bit draw
    differs between seed and seed + 1, so c_q, c_k and c_v of a layer come out equal to within
    1.5e-3.  With q and k that close every query's score with its own key is |y|^2 / sqrt(D) = 11.3
    and the initial attention is all but one-hot on the diagonal.  That is the reference's initial
    state, reproduced here as it is.

    The reference starts c_proj and mlp_proj at zero, which makes the gradient into attention exactly
    zero at the first step; ``test_init`` replaces those zeros by uniform(-0.01, 0.01) with seeds
    12345, 12346, ... as the reference's own forward test does (test_forward.mojo:48-63)."""
    C, V, L = cfg.n_embd, cfg.vocab_size, cfg.n_layer
    kv = cfg.n_kv_head * cfg.head_dim
    mlp = MLP_EXPANSION * C
    s = float(np.float32(math.sqrt(3.0) * C ** -0.5))
    seed, tseed = 42, 12345
    w: Dict[str, torch.Tensor] = {}

    def put(name, arr, shape):
        w[name] = torch.from_numpy(np.ascontiguousarray(arr).reshape(shape)).to(device)

    put("wte", fill_normal(seed, 1.0, V * C), (V, C)); seed += 1
    put("lm_head", fill_normal(seed, 0.001, V * C), (V, C)); seed += 1
    w["resid_lambdas"] = torch.full((L,), 1.0, device=device)
    w["x0_lambdas"] = torch.full((L,), 0.1, device=device)
    for i in range(L):
        put(f"c_q.{i}", fill_uniform(seed, -s, s, C * C), (C, C)); seed += 1
        put(f"c_k.{i}", fill_uniform(seed, -s, s, kv * C), (kv, C)); seed += 1
        put(f"c_v.{i}", fill_uniform(seed, -s, s, kv * C), (kv, C)); seed += 1
        if test_init:
            put(f"c_proj.{i}", fill_uniform(tseed, -0.01, 0.01, C * C), (C, C)); tseed += 1
        else:
            w[f"c_proj.{i}"] = torch.zeros(C, C, device=device)
        put(f"c_fc.{i}", fill_uniform(seed, -s, s, mlp * C), (mlp, C)); seed += 1
        if test_init:
            put(f"mlp_proj.{i}", fill_uniform(tseed, -0.01, 0.01, C * mlp), (C, mlp)); tseed += 1
        else:
            w[f"mlp_proj.{i}"] = torch.zeros(C, mlp, device=device)
        if cfg.has_ve(i):
            put(f"value_embeds.{i}", fill_uniform(seed, -s, s, V * kv), (V, kv)); seed += 1
            w[f"ve_gate.{i}"] = torch.zeros(cfg.n_kv_head, VE_GATE_CHANNELS, device=device)
    return w


# --------------------------------------------------------------------------------------------
# attention back ends
# --------------------------------------------------------------------------------------------
class LibraryAttention:
    """RoPE + per-head RMSNorm + attention through libarattn.so: the prologue kernel
    (ar_qk_norm_rope_cast) writes the rotated, normalised bf16 q, k and the bf16 v; ar_attn_fwd runs
    on them; ar_attn_bwd reads the saved rotated tensors and returns dq, dk with rope_bwd applied and
    the normalisation passed straight through (the reference's flow, model.mojo:937-964)."""

    def __init__(self, cfg: GPTConfig, seq_len: int, device, grad_dtype=torch.bfloat16):
        cos, sin = precompute_rope(seq_len, cfg.head_dim)
        self.tables = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        self.grad_dtype = grad_dtype
        self.events: List = []          # (start, end) CUDA events of every call, for the time share

    def _timed(self, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        self.events.append((e0, e1))
        return out

    def forward(self, q, k, v, window: int):
        """q, k, v: [B, T, H, D] (fp32 or bf16), un-rotated.  Returns (o bf16 [B,T,H,D], ctx)."""
        import ctypes  # noqa: F401  (the binding below is ctypes)

        from . import _lib
        from .attention import AttnParams, attn_fwd

        def run():
            B, T, H, D = q.shape
            q_rot, k_rot, v_b = (torch.empty(B, T, H, D, device=q.device, dtype=torch.bfloat16) for _ in range(3))
            rms_q = torch.empty(B, T, H, device=q.device, dtype=torch.float32)
            rms_k = torch.empty_like(rms_q)
            dt = _lib.AR_F32 if q.dtype == torch.float32 else _lib.AR_BF16
            assert k.dtype == q.dtype and v.dtype == q.dtype and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
            with torch.cuda.device(q.device):
                _lib.check(_lib.lib().ar_qk_norm_rope_cast(
                    q_rot.data_ptr(), k_rot.data_ptr(), v_b.data_ptr(), rms_q.data_ptr(), rms_k.data_ptr(),
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), dt, self.tables[0].data_ptr(), self.tables[1].data_ptr(),
                    B * T, H, D, T, NORM_EPS, torch.cuda.current_stream(q.device).cuda_stream))
            o, lse = attn_fwd(q_rot, k_rot, v_b, AttnParams(window=window))
            return o, dict(q_rot=q_rot, k_rot=k_rot, v=v_b, o=o, lse=lse, rms_q=rms_q, rms_k=rms_k, window=window)

        return self._timed(run)

    def backward(self, ctx, d_o):
        """Returns (dq, dk, dv) [B,T,H,D]: dq, dk with rope_bwd applied and the per-head normalisation
        passed straight through."""
        from .attention import AttnParams, attn_bwd

        def run():
            p = AttnParams(window=ctx["window"], rope=self.tables, q_rot=ctx["q_rot"], k_rot=ctx["k_rot"],
                           grad_dtype=self.grad_dtype)
            do = d_o.to(torch.bfloat16).contiguous()
            dq, dk, dv, _ = attn_bwd(ctx["q_rot"], ctx["k_rot"], ctx["v"], ctx["o"], do, ctx["lse"], p)
            return dq, dk, dv

        return self._timed(run)

    def attention_ms(self) -> float:
        """Device time of all calls since the last reset (synchronises)."""
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in self.events)
        self.events = []
        return ms


# --------------------------------------------------------------------------------------------
# the step
# --------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, dtype=torch.float32):
    """ops.mojo:61-104 on the last axis.  Returns (y, rms) with rms = sqrt(mean(x^2) + eps)."""
    xf = x.to(dtype)
    rms = torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + NORM_EPS)
    return xf / rms, rms


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, rms: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """ops.mojo:1039-1086: dx = (dy - x * dot(dy, x) / (dim * rms^2)) / rms."""
    dy, x = dy.to(dtype), x.to(dtype)
    dot = (dy * x).sum(-1, keepdim=True)
    return (dy - x * dot / (x.shape[-1] * rms * rms)) / rms


@dataclass
class TrainStep:
    """One forward + backward of the model on `ids`, `targets` ([B, T] int64).  Gradients accumulate in
    ``grads`` (fp32, same keys as ``weights``); ``zero_grads`` clears them."""
    cfg: GPTConfig
    weights: Dict[str, torch.Tensor]
    attention: object
    reference_quirks: bool = True
    compute_dtype: torch.dtype = torch.bfloat16      # operand type of the matmuls (accumulation is fp32)
    master_dtype: torch.dtype = torch.float32        # residual stream, saved activations, gradients
    projections: str = "torch"                       # "library": the matmuls through ar_linear_* (bf16 operands)
    grads: Dict[str, torch.Tensor] = field(default_factory=dict)
    process_group: Optional[object] = None
    _pending: List = field(default_factory=list)

    def __post_init__(self):
        if not self.grads:
            self.grads = {k: torch.zeros_like(v) for k, v in self.weights.items()}

    # ---- helpers -------------------------------------------------------------------------
    def _mm(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """a @ b with operands in the compute dtype, result in the master dtype."""
        return (a.to(self.compute_dtype) @ b.to(self.compute_dtype)).to(self.master_dtype)

    def _library(self, *ts: torch.Tensor) -> bool:
        return self.projections == "library" and all(t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) for t in ts)

    def _lin(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """linear_fwd (ops.mojo:110): x [M, K] times weight [N, K] transposed."""
        if not self._library(x, weight):
            return self._mm(x, weight.t())
        from . import ops
        (M, K), N = x.shape, weight.shape[0]
        y = torch.empty(M, N, device=x.device, dtype=self.master_dtype)
        ops.linear_fwd(y, x.contiguous(), weight.to(x.dtype), M, N, K)
        return y

    def _lin_dx(self, dy: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """linear_bwd_dx (ops.mojo:870): dy [M, N] times weight [N, K]."""
        if not self._library(dy, weight):
            return self._mm(dy, weight)
        from . import ops
        (M, N), K = dy.shape, weight.shape[1]
        dx = torch.empty(M, K, device=dy.device, dtype=self.master_dtype)
        ops.linear_bwd_dx(dx, dy.contiguous(), weight.to(dy.dtype), M, N, K)
        return dx

    def _lin_dw(self, name: str, dy: torch.Tensor, x: torch.Tensor) -> None:
        """linear_bwd_dw (ops.mojo:953): grads[name] [N, K] += dy [M, N] transposed times x [M, K]."""
        gw = self.grads[name]
        if not self._library(dy, x) or gw.dtype != torch.float32:
            gw += self._mm(dy.t(), x)
            return
        from . import ops
        (M, N), K = dy.shape, x.shape[1]
        ops.linear_bwd_dw(gw, dy.contiguous(), x.to(dy.dtype).contiguous(), M, N, K)

    def zero_grads(self):
        for g in self.grads.values():
            g.zero_()

    def _layer_grad_names(self, i: int) -> List[str]:
        names = [f"c_q.{i}", f"c_k.{i}", f"c_v.{i}", f"c_proj.{i}", f"c_fc.{i}", f"mlp_proj.{i}"]
        if self.cfg.has_ve(i):
            names += [f"value_embeds.{i}", f"ve_gate.{i}"]
        return names

    def _allreduce_async(self, names: List[str]):
        """One bucket: the named gradients flattened into one buffer, summed over the ranks."""
        if self.process_group is None:
            return
        import torch.distributed as dist
        flat = torch.cat([self.grads[n].reshape(-1) for n in names])
        work = dist.all_reduce(flat, group=self.process_group if self.process_group is not True else None, async_op=True)
        self._pending.append((work, flat, names))

    def finish_allreduce(self, average: bool = True):
        import torch.distributed as dist
        world = dist.get_world_size() if self.process_group is not None else 1
        for work, flat, names in self._pending:
            work.wait()
            off = 0
            for n in names:
                g = self.grads[n]
                g.copy_(flat[off:off + g.numel()].view_as(g))
                if average:
                    g.div_(world)
                off += g.numel()
        self._pending = []

    # ---- forward ---------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.weights
        B, T = ids.shape
        H, D, C = cfg.n_head, cfg.head_dim, cfg.n_embd
        flat = ids.reshape(-1)
        sv: Dict = {"ids": flat, "targets": targets.reshape(-1), "B": B, "T": T, "layers": []}
        emb = w["wte"][flat]
        x, rms_emb = rmsnorm(emb, self.master_dtype)
        sv["emb"], sv["rms_emb"] = emb, rms_emb
        x0 = x
        sv["x0"] = x0
        for i in range(cfg.n_layer):
            L: Dict = {}
            L["x_prev"] = x
            x = w["resid_lambdas"][i] * x + w["x0_lambdas"][i] * x0
            L["x"] = x
            xn, L["rms_attn"] = rmsnorm(x, self.master_dtype)
            L["xn"] = xn
            q = self._lin(xn, w[f"c_q.{i}"])
            k = self._lin(xn, w[f"c_k.{i}"])
            v = self._lin(xn, w[f"c_v.{i}"])
            if cfg.has_ve(i):
                ve = w[f"value_embeds.{i}"][flat]                                               # [BT, kv]
                gate = 2.0 * torch.sigmoid(xn[:, :VE_GATE_CHANNELS] @ w[f"ve_gate.{i}"].t())    # [BT, H]
                v = (v.view(-1, H, D) + gate.unsqueeze(-1) * ve.view(-1, H, D)).reshape(-1, H * D)
                L["ve"], L["gate"] = ve, gate
            L["q_pre"], L["k_pre"] = q, k
            o, L["ctx"] = self.attention.forward(q.view(B, T, H, D).contiguous(), k.view(B, T, H, D).contiguous(),
                                                 v.view(B, T, H, D).contiguous(), cfg.window_size(i))
            o = o.reshape(-1, C).to(self.master_dtype)
            L["o"] = o
            x = x + self._lin(o, w[f"c_proj.{i}"])
            L["x_mid"] = x
            xn2, L["rms_mlp"] = rmsnorm(x, self.master_dtype)
            L["xn2"] = xn2
            hdn = self._lin(xn2, w[f"c_fc.{i}"])
            L["h"] = hdn
            act = torch.relu(hdn).pow(2)
            L["act"] = act
            x = x + self._lin(act, w[f"mlp_proj.{i}"])
            sv["layers"].append(L)
        sv["x_pre_final"] = x
        xf, sv["rms_final"] = rmsnorm(x, self.master_dtype)
        sv["x_final"] = xf
        raw = self._lin(xf, w["lm_head"])
        capped = SOFTCAP * torch.tanh(raw / SOFTCAP)
        sv["raw"], sv["capped"] = raw, capped
        loss = torch.nn.functional.cross_entropy(capped, sv["targets"])
        self._saved = sv
        return loss

    # ---- backward --------------------------------------------------------------------------
    def backward(self, loss_scale: float = 1.0):
        cfg, w, g, sv = self.cfg, self.weights, self.grads, self._saved
        quirks = self.reference_quirks
        B, T = sv["B"], sv["T"]
        H, D = cfg.n_head, cfg.head_dim
        BT = B * T
        ids = sv["ids"]
        probs = torch.softmax(sv["capped"], dim=-1)
        probs[torch.arange(BT, device=probs.device), sv["targets"]] -= 1.0
        dlog = probs * (loss_scale / BT)          # w.r.t. the capped logits (mean over tokens, as mean_reduce does)
        if not quirks:
            dlog = dlog * (1.0 - torch.tanh(sv["raw"] / SOFTCAP).pow(2))
        self._lin_dw("lm_head", dlog, sv["x_final"])
        dx = self._lin_dx(dlog, w["lm_head"])
        dx = rmsnorm_bwd(dx, sv["x_pre_final"], sv["rms_final"], self.master_dtype)
        dx0 = torch.zeros_like(dx)
        for i in reversed(range(cfg.n_layer)):
            L = sv["layers"][i]
            # MLP
            self._lin_dw(f"mlp_proj.{i}", dx, L["act"])
            dact = self._lin_dx(dx, w[f"mlp_proj.{i}"])
            dh = 2.0 * L["h"] * dact * (L["h"] > 0)
            self._lin_dw(f"c_fc.{i}", dh, L["xn2"])
            dxn2 = self._lin_dx(dh, w[f"c_fc.{i}"])
            dx = dx + rmsnorm_bwd(dxn2, L["x"] if quirks else L["x_mid"], L["rms_mlp"], self.master_dtype)
            # attention
            self._lin_dw(f"c_proj.{i}", dx, L["o"])
            d_o = self._lin_dx(dx, w[f"c_proj.{i}"])
            dq, dk, dv = self.attention.backward(L["ctx"], d_o.view(B, T, H, D))
            dq, dk, dv = (t.reshape(BT, H * D).to(self.master_dtype) for t in (dq, dk, dv))
            if not quirks:
                # the per-head normalisation: rotation and normalisation commute, so its backward can
                # be taken on the un-rotated side, after rope_bwd, with y = q / rms
                for grad, pre, rms in ((dq, L["q_pre"], L["ctx"]["rms_q"]), (dk, L["k_pre"], L["ctx"]["rms_k"])):
                    r = rms.reshape(BT, H, 1)
                    y = pre.view(BT, H, D) / r
                    gv = grad.view(BT, H, D)
                    gv.copy_((gv - y * (gv * y).mean(-1, keepdim=True)) / r)
            xn = L["xn"]
            if cfg.has_ve(i):
                dvh = dv.view(BT, H, D)
                dve = (L["gate"].unsqueeze(-1) * dvh).reshape(BT, H * D)
                dgate = (L["ve"].view(BT, H, D) * dvh).sum(-1)                                   # [BT, H]
                g[f"value_embeds.{i}"].index_add_(0, ids, dve)
            self._lin_dw(f"c_q.{i}", dq, xn)
            self._lin_dw(f"c_k.{i}", dk, xn)
            self._lin_dw(f"c_v.{i}", dv, xn)
            dxn = self._lin_dx(dq, w[f"c_q.{i}"]) + self._lin_dx(dk, w[f"c_k.{i}"]) + self._lin_dx(dv, w[f"c_v.{i}"])
            if cfg.has_ve(i):
                dz = dgate * L["gate"] * (1.0 - L["gate"] / 2.0)
                g[f"ve_gate.{i}"] += dz.t() @ xn[:, :VE_GATE_CHANNELS]
                dxn[:, :VE_GATE_CHANNELS] += dz @ w[f"ve_gate.{i}"]
            dx = dx + rmsnorm_bwd(dxn, L["x"], L["rms_attn"], self.master_dtype)
            # learned residual: x = sa * x_prev + sb * x0
            g["resid_lambdas"][i] += (dx * (L["x"] if quirks else L["x_prev"])).sum()
            g["x0_lambdas"][i] += (dx * sv["x0"]).sum()
            if not quirks:
                dx0 = dx0 + w["x0_lambdas"][i] * dx
            dx = w["resid_lambdas"][i] * dx
            self._allreduce_async(self._layer_grad_names(i))
        if not quirks:
            dx = rmsnorm_bwd(dx + dx0, sv["emb"], sv["rms_emb"], self.master_dtype)
        g["wte"].index_add_(0, ids, dx)
        self._allreduce_async(["wte", "lm_head", "resid_lambdas", "x0_lambdas"])
        self._saved = None

    def step(self, ids: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0) -> torch.Tensor:
        loss = self.forward(ids, targets)
        self.backward(loss_scale)
        self.finish_allreduce()
        return loss
