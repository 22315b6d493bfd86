"""Layers: the generated set (Source/Public/Oa/Ml/Nn/Layers.h:7-28) and the manual Transformer family
(Source/Private/Oa/Ml/Nn/{Linear,Embedding,LayerNorm,RmsNorm,Rope,Ffn,Attention,Transformer}).

Checkpoint names follow the reference: `weight` / `bias` on Linear, LayerNorm, RmsNorm, Embedding;
`q_proj k_proj v_proj out_proj` under attention; `ln_attn attention ln_ffn ffn1 ffn2` (or `moe`) under a block;
`norm gate up down` under OaFfn.
"""
from __future__ import annotations

import torch

import math
from typing import Optional

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from .. import autograd as AG
from .. import fn_fused as FF
from ..module import OaModule


class OaIdentity(OaModule):
    def Forward(self, x):
        return x


class OaRelu(OaModule):
    def Forward(self, x):
        return F.Relu(x)


class OaGelu(OaModule):
    def Forward(self, x):
        return F.Gelu(x)


class OaSilu(OaModule):
    def Forward(self, x):
        return F.Silu(x)


class OaSoftmax(OaModule):
    def Forward(self, x):
        return F.Softmax(x)


class OaFlatten(OaModule):
    def Forward(self, x):
        return x.Reshape([x.Size(0), x.NumElements() // x.Size(0)])


class OaDropout(OaModule):
    def __init__(self, p: float = 0.1):
        super().__init__()
        self.P = p

    def Forward(self, x):
        return F.Dropout(x, self.P, self.IsTraining())


class OaSequential(OaModule):
    def __init__(self, *modules):
        super().__init__()
        for i, m in enumerate(modules):
            self.RegisterModule(str(i), m)

    def Add(self, module: OaModule) -> "OaSequential":
        self.RegisterModule(str(len(self._children)), module)
        return self

    def Forward(self, x):
        for _, m in self._children:
            x = m.Forward(x)
        return x


class OaLinear(OaModule):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, init_std: Optional[float] = None):
        super().__init__()
        self.InFeatures, self.OutFeatures = in_features, out_features
        w = F.RandXavier([out_features, in_features]) if init_std is None else F.RandN([out_features, in_features], std=init_std)
        self.Weight = self.RegisterParameter("weight", w)
        self.Bias = self.RegisterParameter("bias", F.Zeros([out_features])) if bias else None

    def Forward(self, x):
        return F.Linear(x, self.Weight.Data, self.Bias.Data if self.Bias else None)


class OaEmbedding(OaModule):
    def __init__(self, num_embeddings: int, embedding_dim: int, init_std: Optional[float] = None):
        super().__init__()
        self.NumEmbeddings, self.EmbeddingDim = num_embeddings, embedding_dim
        self.Weight = self.RegisterParameter("weight", F.RandN([num_embeddings, embedding_dim], std=init_std))

    def Forward(self, ids):
        return F.Gather(self.Weight.Data, ids)


class OaLayerNorm(OaModule):
    def __init__(self, normalized_shape: int, eps: float = 1e-5):
        super().__init__()
        self.Eps = eps
        self.Weight = self.RegisterParameter("weight", F.Ones([normalized_shape]))
        self.Bias = self.RegisterParameter("bias", F.Zeros([normalized_shape]))

    def Forward(self, x):
        return F.LayerNorm(x, self.Weight.Data, self.Bias.Data, self.Eps)


class OaRmsNorm(OaModule):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.Eps = eps
        self.Weight = self.RegisterParameter("weight", F.Ones([dim]))

    def Forward(self, x):
        return F.RmsNorm(x, self.Weight.Data, self.Eps)


class OaRoPE(OaModule):
    """Rotate-half rotary embedding, theta = 1e4 by default (Source/Private/Oa/Ml/Nn/Rope/Rope.cpp:16-63)."""

    def __init__(self, head_dim: int, max_seq: int = 0, theta: float = 10000.0):
        super().__init__()
        self.HeadDim, self.Theta, self.MaxSeq = head_dim, theta, max_seq

    def Apply(self, x: OaMatrix, heads: int, seq: int, pos_offset: int = 0) -> OaMatrix:
        return F.RoPE(x, heads, self.HeadDim, seq, pos_offset, self.Theta)

    def Forward(self, x):
        raise RuntimeError("OaRoPE: call Apply(x, heads, seq)")


class OaSwiGLU(OaModule):
    def Forward(self, x):
        return F.Swiglu(x)


class OaAttentionBackend:
    Auto, Standard, Flash = 0, 1, 2


class OaAttentionMode:
    Causal, Bidirectional = 0, 1


class OaMultiHeadAttention(OaModule):
    """Causal multi-head self-attention with q/k/v/out Linear children.

    One packed QKV GEMM feeds the tiled tensor-core attention kernel directly (no SplitHeads / MergeHeads copies).
    Unlike the reference (Flash only for inference, S <= 1024, FP32; MultiHeadAttention.cpp:119-130) the flash path
    is the training path for any sequence length.  `Backend=Standard` keeps the materialised
    Bmm -> SoftmaxScaledMasked -> Bmm route for differential tests.
    """

    def __init__(self, d_model: int, num_heads: int, max_seq: int = 0, bias: bool = True, causal: bool = True,
                 rope_theta: float = 0.0, init_std: Optional[float] = None, backend: int = OaAttentionBackend.Auto):
        super().__init__()
        assert d_model % num_heads == 0
        self.DModel, self.NumHeads, self.HeadDim = d_model, num_heads, d_model // num_heads
        self.Causal, self.RopeTheta, self.Backend = causal, rope_theta, backend
        # q, k, v are row slices of one packed [3D, D] tensor so that the packed projection is copy-free
        packed = F.RandXavier([3 * d_model, d_model]) if init_std is None else F.RandN([3 * d_model, d_model], std=init_std)
        pt = packed.Tensor()
        pb = F.Zeros([3 * d_model]).Tensor() if bias else None
        self.QProj, self.KProj, self.VProj = (OaLinear.__new__(OaLinear) for _ in range(3))
        for i, (lin, nm) in enumerate(((self.QProj, "q_proj"), (self.KProj, "k_proj"), (self.VProj, "v_proj"))):
            OaModule.__init__(lin)
            lin.InFeatures = lin.OutFeatures = d_model
            lin.Weight = lin.RegisterParameter("weight", OaMatrix(pt[i * d_model:(i + 1) * d_model]))
            lin.Bias = lin.RegisterParameter("bias", OaMatrix(pb[i * d_model:(i + 1) * d_model])) if bias else None
            self.RegisterModule(nm, lin)
        self.OutProj = self.RegisterModule("out_proj", OaLinear(d_model, d_model, bias, init_std))

    Plan = None      # OaBlockPlan of the enclosing block (None: every fused engine)

    def ProjectQkv(self, x: OaMatrix) -> OaMatrix:
        ws = [self.QProj.Weight.Data, self.KProj.Weight.Data, self.VProj.Weight.Data]
        bs = [l.Bias.Data if l.Bias else None for l in (self.QProj, self.KProj, self.VProj)]
        if self.Plan is not None and not self.Plan.PackedQkv:          # portable lowering: three products, joined
            return F.Concat([F.Linear(x, w, b) for w, b in zip(ws, bs)], -1)
        return FF.PackedProjection(x, ws, bs, "PackedLinear3")

    def _flash_capable(self) -> bool:
        if self.Backend == OaAttentionBackend.Standard:
            return False
        w = self.OutProj.Weight.Tensor()
        return not (w.is_cuda and w.dtype == torch.bfloat16 and self.HeadDim not in (64, 128))

    def _use_flash(self) -> bool:
        if self.Plan is not None and not self.Plan.FlashAttention:
            return False
        if self.Backend == OaAttentionBackend.Standard:
            return False
        w = self.OutProj.Weight.Tensor()
        if w.is_cuda and w.dtype == torch.bfloat16 and self.HeadDim not in (64, 128):
            return False          # the tensor-core kernel is built for head dims 64 and 128; others take the materialised path
        return True

    def Attend(self, qkv: OaMatrix, batch: int, seq: int, pos_offset: int = 0, mask: Optional[OaMatrix] = None) -> OaMatrix:
        """`mask`, when given, is an additive [B*H*S, S] (or [S, S]) mask: it takes the materialised path and replaces the
        causal mask (MultiHeadAttention::ForwardMasked of the reference)."""
        if mask is None and self._use_flash():
            return F.FlashAttentionPacked(qkv, batch, seq, self.NumHeads, self.HeadDim, causal=self.Causal,
                                          rope_theta=self.RopeTheta, pos_offset=pos_offset, consume_input=True)
        D, H = self.DModel, self.NumHeads
        q, k, v = F.Split(qkv, [D, D, D], -1)
        if self.RopeTheta > 0:
            q = F.RoPE(q, H, self.HeadDim, seq, pos_offset, self.RopeTheta)
            k = F.RoPE(k, H, self.HeadDim, seq, pos_offset, self.RopeTheta)
        qh, kh, vh = (F.SplitHeads(t, batch, seq, H) for t in (q, k, v))
        scores = F.Bmm(qh, F.Transpose(kh, 1, 2))
        if mask is None and self.Causal:
            mask = F.CausalMask(seq, scores.Dtype())       # [S, S], repeated over batch and heads by the kernel
        probs = F.SoftmaxScaledMasked(scores, 1.0 / math.sqrt(self.HeadDim), mask)
        return F.MergeHeads(F.Bmm(probs, vh), batch, seq, H)

    def ForwardMasked(self, x: OaMatrix, additive_mask: OaMatrix, batch: Optional[int] = None, seq: Optional[int] = None,
                      residual: Optional[OaMatrix] = None) -> OaMatrix:
        return self.Forward(x, batch, seq, residual, 0, additive_mask)

    def Forward(self, x: OaMatrix, batch: Optional[int] = None, seq: Optional[int] = None, residual: Optional[OaMatrix] = None,
                pos_offset: int = 0, mask: Optional[OaMatrix] = None) -> OaMatrix:
        """x: [B*S, D] (pass batch, seq) or [B, S, D]."""
        shape3 = x.Rank() == 3
        if shape3:
            batch, seq = x.Size(0), x.Size(1)
            x = x.Reshape([batch * seq, self.DModel])
        a = self.Attend(self.ProjectQkv(x), batch, seq, pos_offset, mask)
        o = self.OutProj
        y = F.Linear(a, o.Weight.Data, o.Bias.Data if o.Bias else None, residual=residual)
        return y.Reshape([batch, seq, self.DModel]) if shape3 else y


class OaFfn(OaModule):
    """Pre-norm gated FFN with residual: x + Down(Swiglu([Gate; Up] RmsNorm(x)))  (Source/Private/Oa/Ml/Nn/Ffn/Ffn.cpp:49-76)."""

    def __init__(self, d_model: int, d_ff: int, eps: float = 1e-6, init_std: Optional[float] = None):
        super().__init__()
        self.Norm = self.RegisterModule("norm", OaRmsNorm(d_model, eps))
        packed = (F.RandXavier([2 * d_ff, d_model]) if init_std is None else F.RandN([2 * d_ff, d_model], std=init_std)).Tensor()
        self.Gate, self.Up = OaLinear.__new__(OaLinear), OaLinear.__new__(OaLinear)
        for i, (lin, nm) in enumerate(((self.Gate, "gate"), (self.Up, "up"))):
            OaModule.__init__(lin)
            lin.InFeatures, lin.OutFeatures, lin.Bias = d_model, d_ff, None
            lin.Weight = lin.RegisterParameter("weight", OaMatrix(packed[i * d_ff:(i + 1) * d_ff]))
            self.RegisterModule(nm, lin)
        self.Down = self.RegisterModule("down", OaLinear(d_ff, d_model, False, init_std))

    Plan = None      # OaBlockPlan of the enclosing block (None: every fused engine)

    def Forward(self, x):
        h = self.Norm.Forward(x)
        return _ffn_swiglu(self.Plan, h, self.Gate.Weight.Data, self.Up.Weight.Data, self.Down.Weight.Data, x)


def _ffn_swiglu(plan, h, gate, up, down, residual=None):
    if plan is not None and not plan.GatedFfn:                         # portable lowering
        return F.Linear(F.Mul(F.Silu(F.Linear(h, gate)), F.Linear(h, up)), down, None, residual=residual)
    return FF.FfnSwiglu(h, gate, up, down, residual=residual)


def _ffn_gelu(plan, h, w1, b1, w2, b2, residual=None):
    if plan is not None and not plan.GemmEpilogue:                     # portable lowering: activation as its own operation
        return F.Linear(F.Gelu(F.Linear(h, w1, b1)), w2, b2, residual=residual)
    return FF.FfnGelu(h, w1, b1, w2, b2, residual=residual)


class OaTransformerBlock(OaModule):
    """Pre-norm block: x + Attn(Norm(x)); then x + FFN(Norm(x)) with a fused Linear+GELU FFN, an OaFfn-style
    SwiGLU FFN, or a sparse MoE layer (Source/Private/Oa/Ml/Nn/Transformer/Transformer.cpp:37-185)."""

    def __init__(self, d_model: int, d_ff: int, seq_len: int, num_heads: int, eps: float = 1e-5, *, norm: str = "layer",
                 ffn: str = "gelu", bias: bool = True, rope_theta: float = 0.0, moe=None, init_std: Optional[float] = None,
                 attention_backend: int = OaAttentionBackend.Auto):
        super().__init__()
        self.DModel, self.SeqLen, self.FfnKind = d_model, seq_len, ffn
        self.AdaptiveModulation, self.ConditionDim = None, 0
        mk_norm = (lambda: OaLayerNorm(d_model, eps)) if norm == "layer" else (lambda: OaRmsNorm(d_model, eps))
        self.Moe = None
        if moe is not None:
            self.Moe = self.RegisterModule("moe", moe)
        elif ffn == "gelu":
            self.LnFfn = self.RegisterModule("ln_ffn", mk_norm())
            self.Ffn1 = self.RegisterModule("ffn1", OaLinear(d_model, d_ff, bias, init_std))
            self.Ffn2 = self.RegisterModule("ffn2", OaLinear(d_ff, d_model, bias, init_std))
        else:
            self.Ffn = self.RegisterModule("ffn", OaFfn(d_model, d_ff, eps, init_std))
        self.LnAttn = self.RegisterModule("ln_attn", mk_norm())
        self.Attention = self.RegisterModule("attention", OaMultiHeadAttention(d_model, num_heads, seq_len, bias, True, rope_theta,
                                                                               init_std, attention_backend))

    # ---- attention mode, sequence length, adaptive conditioning (Transformer.cpp:93-147, 171-185)
    def SetAttentionMode(self, mode: int) -> None:
        self.Attention.Causal = mode == OaAttentionMode.Causal

    def SetSeqLen(self, seq_len: int) -> None:
        if seq_len <= 0:
            raise ValueError("sequence length must be positive")
        self.SeqLen = seq_len

    def EnableAdaptiveConditioning(self, condition_dim: int) -> None:
        """AdaLN-Zero: a zero-initialised Linear(condition -> 6*D) yields shift / scale / gate for the attention and FFN
        branches, so an untrained block starts as the identity of its residual path."""
        if condition_dim <= 0:
            raise ValueError("adaptive condition dimension must be positive")
        if self.AdaptiveModulation is not None:
            if self.ConditionDim != condition_dim:
                raise ValueError("adaptive conditioning is already configured with a different dimension")
            return
        self.ConditionDim = condition_dim
        lin = OaLinear(condition_dim, 6 * self.DModel)
        lin.Weight.Data.Tensor().zero_()
        self.AdaptiveModulation = self.RegisterModule("adaptive_modulation", lin)

    def ForwardMasked(self, x: OaMatrix, additive_mask: OaMatrix, batch: Optional[int] = None, seq: Optional[int] = None) -> OaMatrix:
        return self.Forward(x, batch, seq, 0, additive_mask)

    def BlockPlan(self):
        """The engines this block runs with, from the native fusion planner (planned once per block description)."""
        from .block_plan import PlanTransformerBlock
        kind = "moe" if self.Moe is not None else ("gelu" if self.FfnKind == "gelu" else "swiglu")
        d_ff = self.Ffn1.OutFeatures if kind == "gelu" else (self.Ffn.Down.InFeatures if kind == "swiglu" else 0)
        plan = PlanTransformerBlock(self.DModel, d_ff, kind, self.Attention.OutProj.Bias is not None, self.Attention._flash_capable(),
                                    training=self.IsTraining() if hasattr(self, "IsTraining") else True)
        self.Attention.Plan = plan
        if self.Moe is None and kind == "swiglu":
            self.Ffn.Plan = plan
        return plan

    def _ffn_delta(self, h: OaMatrix) -> OaMatrix:
        if self.Moe is not None:
            return self.Moe.Forward(h)
        plan = self.BlockPlan()
        if self.FfnKind == "gelu":
            return _ffn_gelu(plan, h, self.Ffn1.Weight.Data, self.Ffn1.Bias.Data if self.Ffn1.Bias else None, self.Ffn2.Weight.Data,
                             self.Ffn2.Bias.Data if self.Ffn2.Bias else None)
        f = self.Ffn
        return _ffn_swiglu(plan, h, f.Gate.Weight.Data, f.Up.Weight.Data, f.Down.Weight.Data)

    def ForwardConditioned(self, x: OaMatrix, condition: OaMatrix, additive_mask: Optional[OaMatrix] = None) -> OaMatrix:
        """x [B*S, D], condition [B, C]: x + gate_a * Attn(norm(x) * (1 + scale_a) + shift_a), then the same for the FFN."""
        if self.AdaptiveModulation is None:
            raise ValueError("adaptive conditioning must be enabled before ForwardConditioned")
        rows, S, D = x.Size(0), self.SeqLen, self.DModel
        if x.Rank() != 2 or x.Size(1) != D or S <= 0 or rows % S or condition.Rank() != 2 or condition.Size(0) != rows // S \
                or condition.Size(1) != self.ConditionDim:
            raise ValueError("conditioned input must be [B*S, D] with condition [B, C]")
        mod = F.RepeatInterleave(self.AdaptiveModulation.Forward(condition), S, 0)
        sh_a, sc_a, g_a, sh_f, sc_f, g_f = F.Split(mod, [D] * 6, 1)
        h = F.Add(F.Mul(self.LnAttn.Forward(x), F.AddScalar(sc_a, 1.0)), sh_a)
        x = F.Add(x, F.Mul(self.Attention.Forward(h, rows // S, S, mask=additive_mask), g_a))
        h = self.LnFfn.Forward(x) if self.Moe is None and self.FfnKind == "gelu" else (self.Ffn.Norm.Forward(x) if self.Moe is None else x)
        h = F.Add(F.Mul(h, F.AddScalar(sc_f, 1.0)), sh_f)
        return F.Add(x, F.Mul(self._ffn_delta(h), g_f))

    def Forward(self, x: OaMatrix, batch: Optional[int] = None, seq: Optional[int] = None, pos_offset: int = 0,
                mask: Optional[OaMatrix] = None) -> OaMatrix:
        shape3 = x.Rank() == 3
        if shape3:
            batch, seq = x.Size(0), x.Size(1)
            x = x.Reshape([batch * seq, self.DModel])
        if batch is None:
            seq = self.SeqLen
            batch = x.Size(0) // seq
        plan = self.BlockPlan()
        x = self.Attention.Forward(self.LnAttn.Forward(x), batch, seq, residual=x, pos_offset=pos_offset, mask=mask)
        if self.Moe is not None:
            x = self.Moe.Forward(x)
        elif self.FfnKind == "gelu":
            h = self.LnFfn.Forward(x)
            x = _ffn_gelu(plan, h, self.Ffn1.Weight.Data, self.Ffn1.Bias.Data if self.Ffn1.Bias else None, self.Ffn2.Weight.Data,
                          self.Ffn2.Bias.Data if self.Ffn2.Bias else None, residual=x)
        else:
            x = self.Ffn.Forward(x)
        return x.Reshape([batch, seq, self.DModel]) if shape3 else x
