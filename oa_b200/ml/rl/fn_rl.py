"""OaFnRl: advantage estimation, policy distributions, transforms and the RL objectives.

Reference: Source/Public/Oa/Ml/Rl/Gae.h:18-56, Policy.h:34-79, Transform.h:9-33, FnLoss.h:57-117 and their
implementations under Source/Private/Oa/Ml/Rl/{Gae,Policy,Transform}.cpp and Rl/FnLoss/{Ppo,Dqn,Sac}.cpp.
Differentiable paths are compositions of tape-recorded matrix functions; targets (GAE, DQN / SAC bootstrap, PPO clip)
are single fused kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...ops import rl as R
from .. import autograd as AG
from .. import fn_loss as L

LOG_TWO_PI = 1.8378770664093453


# ------------------------------------------------------------------------------------------------------------ GAE
@dataclass
class OaGaeConfig:
    Gamma: float = 0.99
    Lambda: float = 0.95


@dataclass
class OaGaeResult:
    Advantage: Optional[OaMatrix] = None     # [Time, Environments] fp32
    Return: Optional[OaMatrix] = None        # Advantage + Value

    def IsValid(self) -> bool:
        return self.Advantage is not None and self.Return is not None


def _is_f32(m: OaMatrix, shape) -> bool:
    return m is not None and not m.IsEmpty() and m.Tensor().dtype == torch.float32 and tuple(m.Tensor().shape) == tuple(shape)


def _is_u8(m: OaMatrix, shape) -> bool:
    return m is not None and not m.IsEmpty() and m.Tensor().dtype == torch.uint8 and tuple(m.Tensor().shape) == tuple(shape)


def GaeInto(reward, value, next_value, terminated, truncated, out_advantage: OaMatrix, out_return: OaMatrix,
            config: Optional[OaGaeConfig] = None):
    """Allocation-free generalised advantage estimation over a fixed [T, E] rollout.  Returns an OaStatus."""
    from ...core.types import OaStatus, OaStatusCode
    cfg = config or OaGaeConfig()
    shape = tuple(reward.Tensor().shape)
    ok = (len(shape) == 2 and all(_is_f32(m, shape) for m in (reward, value, next_value, out_advantage, out_return))
          and _is_u8(terminated, shape) and _is_u8(truncated, shape) and 0.0 <= cfg.Gamma <= 1.0 and 0.0 <= cfg.Lambda <= 1.0)
    if not ok:
        return OaStatus.Error(OaStatusCode.InvalidArgument, "Gae expects matching [T, E] FP32 fields, UInt8 masks and gamma, lambda in [0, 1]")
    F._ctx_add("RlGae")
    c = lambda m: F._c(m.Tensor())
    R.gae(c(reward), c(value), c(next_value), c(terminated), c(truncated), out_advantage.Tensor(), out_return.Tensor(), cfg.Gamma, cfg.Lambda)
    return OaStatus.Ok()


def Gae(reward, value, next_value, terminated, truncated, config: Optional[OaGaeConfig] = None) -> OaGaeResult:
    adv = OaMatrix(torch.empty_like(reward.Tensor(), dtype=torch.float32))
    ret = OaMatrix(torch.empty_like(reward.Tensor(), dtype=torch.float32))
    st = GaeInto(reward, value, next_value, terminated, truncated, adv, ret, config)
    return OaGaeResult(adv, ret) if st else OaGaeResult()


def NormalizeAdvantages(advantage: OaMatrix, epsilon: float = 1e-8) -> OaMatrix:
    """(A - mean) / (std + eps) over every supplied sample (population standard deviation); target preparation, no tape."""
    F._ctx_add("RlNormalizeAdvantages")
    a = advantage.Tensor().float()
    mean = a.mean()
    std = (a - mean).square().mean().sqrt()
    return OaMatrix((a - mean) / (std + epsilon))


# ------------------------------------------------------------------------------------------------------- policies
@dataclass
class OaRlPolicyResult:
    Action: Optional[OaMatrix] = None            # Int32 [E]
    LogProbability: Optional[OaMatrix] = None    # fp32 [E]
    Entropy: Optional[OaMatrix] = None           # fp32 [E]
    Value: Optional[OaMatrix] = None             # fp32 [E]

    def IsValid(self) -> bool:
        return all(m is not None and not m.IsEmpty() for m in (self.Action, self.LogProbability, self.Entropy, self.Value))


@dataclass
class OaRlContinuousPolicyResult:
    Action: Optional[OaMatrix] = None            # fp32 [E, A] inside [minimum, maximum]
    RawAction: Optional[OaMatrix] = None         # fp32 [E, A] before tanh: the stable carrier for re-evaluation
    LogProbability: Optional[OaMatrix] = None
    Entropy: Optional[OaMatrix] = None           # of the base diagonal Gaussian
    Value: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(m is not None and not m.IsEmpty() for m in (self.Action, self.RawAction, self.LogProbability, self.Entropy, self.Value))


def _policy_shape_ok(logits: OaMatrix, value: OaMatrix) -> bool:
    t = logits.Tensor()
    return t.dim() == 2 and t.shape[0] > 0 and t.shape[1] > 1 and t.dtype == torch.float32 and _is_f32(value, (t.shape[0],))


def SampleLogits(logits: OaMatrix, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> OaMatrix:
    """One class index per row of fp32 logits [rows, classes] (OaFnMatrix::SampleLogits, Source/Public/Oa/Core/FnMatrix.h:72).
    Seed 0 draws a fresh seed from the engine's generator; temperature <= 0 is greedy."""
    F._ctx_add("SampleLogits")
    t = F._c(logits.Tensor())
    if top_k > 0 or top_p < 1.0:
        v = t / max(temperature, 1e-6)
        if top_k > 0:
            kth = torch.topk(v, min(top_k, v.shape[1]), dim=1).values[:, -1:]
            v = v.masked_fill(v < kth, float("-inf"))
        if top_p < 1.0:
            sv, si = torch.sort(v, dim=1, descending=True)
            cdf = torch.cumsum(torch.softmax(sv, 1), 1)
            drop = (cdf - torch.softmax(sv, 1)) >= top_p
            v = v.masked_fill(torch.zeros_like(drop).scatter(1, si, drop), float("-inf"))
        t, temperature = v.contiguous(), 1.0
    if seed == 0:
        seed = int(torch.randint(1, 2 ** 62, (1,)).item())
    return OaMatrix(R.sample_categorical(t, seed, max(temperature, 1e-6), greedy=temperature <= 0.0))


def EvaluateCategoricalPolicy(logits: OaMatrix, action: OaMatrix, value: OaMatrix) -> OaRlPolicyResult:
    """log pi(a|s) and entropy of stored actions; gradients flow through the logits."""
    E = logits.Size(0) if logits.Tensor().dim() == 2 else 0
    if not _policy_shape_ok(logits, value) or tuple(action.Tensor().shape) != (E,) or action.Tensor().dtype != torch.int32:
        return OaRlPolicyResult()
    logp_all = F.LogSoftmax(logits, 1)
    selected = F.GatherLastDim(logp_all, F.Reshape(action, [E, 1]))
    prob = F.Exp(logp_all)
    entropy = F.Neg(F.Sum(F.Mul(prob, logp_all), 1))
    return OaRlPolicyResult(action, F.Reshape(selected, [E]), F.Reshape(entropy, [E]), value)


def SampleCategoricalPolicy(logits: OaMatrix, value: OaMatrix, seed: int = 0) -> OaRlPolicyResult:
    if not _policy_shape_ok(logits, value):
        return OaRlPolicyResult()
    return EvaluateCategoricalPolicy(logits, SampleLogits(logits, 1.0, 0, 1.0, seed), value)


def _continuous_ok(mean, log_std, value, lo, hi, eps) -> bool:
    t = mean.Tensor()
    return (t.dim() == 2 and t.shape[0] > 0 and t.shape[1] > 0 and t.dtype == torch.float32 and _is_f32(log_std, t.shape)
            and _is_f32(value, (t.shape[0],)) and math.isfinite(lo) and math.isfinite(hi) and lo < hi and 0.0 < eps < 1.0)


def EvaluateTanhNormalPolicy(mean, log_stddev, raw_action, value, minimum: float = -1.0, maximum: float = 1.0,
                             epsilon: float = 1e-6) -> OaRlContinuousPolicyResult:
    """Diagonal Gaussian squashed by tanh into [minimum, maximum]; the log-probability carries the Jacobian
    log(scale * (1 - tanh^2 + eps)) per dimension."""
    if not _continuous_ok(mean, log_stddev, value, minimum, maximum, epsilon) or not _is_f32(raw_action, mean.Tensor().shape):
        return OaRlContinuousPolicyResult()
    E = mean.Size(0)
    scale, bias = 0.5 * (maximum - minimum), 0.5 * (maximum + minimum)
    log_std = F.ClampMax(F.ClampMin(log_stddev, -20.0), 2.0)
    std = F.Exp(log_std)
    normalized = F.Div(F.Sub(raw_action, mean), std)
    base = F.Scale(F.AddScalar(F.Add(F.Mul(normalized, normalized), F.Scale(log_std, 2.0)), LOG_TWO_PI), -0.5)
    squashed = F.Tanh(raw_action)
    action = F.AddScalar(F.Scale(squashed, scale), bias)
    jacobian = F.Log(F.AddScalar(F.Scale(F.Mul(squashed, squashed), -1.0), 1.0 + epsilon))
    corrected = F.Sub(base, F.AddScalar(jacobian, math.log(scale)))
    entropy_dim = F.AddScalar(log_std, 0.5 * (1.0 + LOG_TWO_PI))
    return OaRlContinuousPolicyResult(action, raw_action, F.Reshape(F.Sum(corrected, 1), [E]), F.Reshape(F.Sum(entropy_dim, 1), [E]), value)


def SampleTanhNormalPolicy(mean, log_stddev, value, minimum: float = -1.0, maximum: float = 1.0, seed: int = 0,
                           epsilon: float = 1e-6) -> OaRlContinuousPolicyResult:
    """Reparameterised draw raw = mean + exp(log_std) * noise, so gradients reach mean and log_std through the action."""
    if not _continuous_ok(mean, log_stddev, value, minimum, maximum, epsilon):
        return OaRlContinuousPolicyResult()
    log_std = F.ClampMax(F.ClampMin(log_stddev, -20.0), 2.0)
    g = torch.Generator(device=mean.Tensor().device)
    g.manual_seed(seed if seed else int(torch.randint(1, 2 ** 62, (1,)).item()))
    noise = OaMatrix(torch.randn(mean.Tensor().shape, generator=g, device=mean.Tensor().device, dtype=torch.float32))
    raw = F.Add(mean, F.Mul(F.Exp(log_std), noise))
    return EvaluateTanhNormalPolicy(mean, log_std, raw, value, minimum, maximum, epsilon)


# ------------------------------------------------------------------------------------------------------ transforms
def NormalizeObservation(observation, mean, stddev, epsilon: float = 1e-6, clip: float = 10.0) -> OaMatrix:
    out = F.Div(F.Sub(observation, mean), F.AddScalar(stddev, epsilon))
    return F.ClampMax(F.ClampMin(out, -clip), clip) if clip > 0 else out


def ScaleAction(action, source_min: float, source_max: float, target_min: float, target_max: float, clamp: bool = True) -> OaMatrix:
    a = F.ClampMax(F.ClampMin(action, source_min), source_max) if clamp else action
    k = (target_max - target_min) / (source_max - source_min)
    return F.AddScalar(F.Scale(F.AddScalar(a, -source_min), k), target_min)


def ClipReward(reward, minimum: float = -1.0, maximum: float = 1.0) -> OaMatrix:
    return F.ClampMax(F.ClampMin(reward, minimum), maximum)


# ----------------------------------------------------------------------------------------------------------- losses
@dataclass
class OaPpoLossConfig:
    ClipEpsilon: float = 0.2
    ValueCoefficient: float = 0.5
    EntropyCoefficient: float = 0.01


@dataclass
class OaPpoLossResult:
    PolicyLoss: Optional[OaMatrix] = None
    ValueLoss: Optional[OaMatrix] = None
    Entropy: Optional[OaMatrix] = None
    TotalLoss: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(m is not None for m in (self.PolicyLoss, self.ValueLoss, self.Entropy, self.TotalLoss))


@dataclass
class OaDqnLossConfig:
    Discount: float = 0.99


@dataclass
class OaDqnLossResult:
    SelectedQ: Optional[OaMatrix] = None
    TargetQ: Optional[OaMatrix] = None
    Loss: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(m is not None for m in (self.SelectedQ, self.TargetQ, self.Loss))


@dataclass
class OaSacLossConfig:
    Discount: float = 0.99
    EntropyCoefficient: float = 0.2


@dataclass
class OaSacCriticLossResult:
    TargetQ: Optional[OaMatrix] = None
    Q1Loss: Optional[OaMatrix] = None
    Q2Loss: Optional[OaMatrix] = None
    TotalLoss: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(m is not None for m in (self.TargetQ, self.Q1Loss, self.Q2Loss, self.TotalLoss))


def _ppo_inputs_ok(new_lp, old_lp, adv, eps) -> bool:
    shape = tuple(new_lp.Tensor().shape)
    return (len(shape) > 0 and new_lp.NumElements() > 0 and all(_is_f32(m, shape) for m in (new_lp, old_lp, adv))
            and math.isfinite(eps) and 0.0 < eps < 1.0)


def PpoClippedPolicyBwd(new_lp, old_lp, adv, clip_epsilon: float = 0.2) -> Optional[OaMatrix]:
    if not _ppo_inputs_ok(new_lp, old_lp, adv, clip_epsilon):
        return None
    F._ctx_add("RlPpoClipBwd")
    c = lambda m: F._c(m.Tensor())
    return OaMatrix(R.ppo_clip(c(new_lp), c(old_lp), c(adv), clip_epsilon, True))


def PpoClippedPolicy(new_lp, old_lp, adv, clip_epsilon: float = 0.2) -> Optional[OaMatrix]:
    """Scalar -mean(min(ratio A, clamp(ratio, 1 +- eps) A)); only the new log-probability is differentiated."""
    if not _ppo_inputs_ok(new_lp, old_lp, adv, clip_epsilon):
        return None
    L._set("ppo_clipped_policy")
    c = lambda m: F._c(m.Tensor())
    per = R.ppo_clip(c(new_lp), c(old_lp), c(adv), clip_epsilon, False)
    out = OaMatrix(K.mean_f32(per.reshape(-1)))

    def back(g):
        grad = R.ppo_clip(c(new_lp), c(old_lp), c(adv), clip_epsilon, True)
        return (grad if L._is_one(g) else K.binary("mul", grad, g.reshape(1).to(grad.dtype)), None, None)

    return AG.attach("PpoClippedPolicy", out, [new_lp, old_lp, adv], back)


def Ppo(new_lp, old_lp, adv, value, target_return, entropy, config: Optional[OaPpoLossConfig] = None) -> OaPpoLossResult:
    cfg = config or OaPpoLossConfig()
    shape = tuple(new_lp.Tensor().shape)
    ok = (math.isfinite(cfg.ValueCoefficient) and math.isfinite(cfg.EntropyCoefficient) and cfg.ValueCoefficient >= 0
          and cfg.EntropyCoefficient >= 0 and _ppo_inputs_ok(new_lp, old_lp, adv, cfg.ClipEpsilon)
          and all(_is_f32(m, shape) for m in (value, target_return, entropy)))
    if not ok:
        return OaPpoLossResult()
    policy = PpoClippedPolicy(new_lp, old_lp, adv, cfg.ClipEpsilon)
    vloss = L.Mse(value, target_return)
    ent = F.Mean(entropy)
    total = F.Sub(F.Add(policy, F.Scale(vloss, cfg.ValueCoefficient)), F.Scale(ent, cfg.EntropyCoefficient))
    L._set("ppo")
    return OaPpoLossResult(policy, vloss, ent, total)


def Dqn(q, action, reward, next_q, terminated, truncated, config: Optional[OaDqnLossConfig] = None) -> OaDqnLossResult:
    """One-step TD objective: SmoothL1(Q(s, a), r + discount * max_a' Q_target(s', a')); termination removes the
    bootstrap, truncation does not.  next_q is target-network data and takes no gradient."""
    cfg = config or OaDqnLossConfig()
    t = q.Tensor()
    B = t.shape[0] if t.dim() == 2 else 0
    ok = (B > 0 and t.dtype == torch.float32 and _is_f32(next_q, t.shape) and _is_f32(reward, (B,)) and _is_u8(terminated, (B,))
          and _is_u8(truncated, (B,)) and tuple(action.Tensor().shape) == (B,) and action.Tensor().dtype == torch.int32
          and 0.0 <= cfg.Discount <= 1.0 and not next_q.RequiresGrad())
    if not ok:
        return OaDqnLossResult()
    F._ctx_add("RlDqnTarget")
    target = OaMatrix(R.dqn_target(F._c(reward.Tensor()), F._c(next_q.Tensor()), F._c(terminated.Tensor()), cfg.Discount))
    selected = F.Reshape(F.GatherLastDim(q, F.Reshape(action, [B, 1])), [B])
    res = OaDqnLossResult(selected, target, L.SmoothL1(selected, target))
    L._set("dqn")
    return res


def SacCritic(q1, q2, reward, next_q1, next_q2, next_log_probability, terminated, truncated,
              config: Optional[OaSacLossConfig] = None) -> OaSacCriticLossResult:
    cfg = config or OaSacLossConfig()
    B = q1.Tensor().shape[0] if q1.Tensor().dim() == 1 else 0
    ok = (B > 0 and all(_is_f32(m, (B,)) for m in (q1, q2, reward, next_q1, next_q2, next_log_probability))
          and _is_u8(terminated, (B,)) and _is_u8(truncated, (B,)) and 0.0 <= cfg.Discount <= 1.0 and cfg.EntropyCoefficient >= 0)
    if not ok:
        return OaSacCriticLossResult()
    F._ctx_add("RlSacTarget")
    c = lambda m: F._c(m.Tensor())
    target = OaMatrix(R.sac_target(c(reward), c(next_q1), c(next_q2), c(next_log_probability), c(terminated), cfg.Discount, cfg.EntropyCoefficient))
    l1, l2 = L.Mse(q1, target), L.Mse(q2, target)
    res = OaSacCriticLossResult(target, l1, l2, F.Add(l1, l2))
    L._set("sac_critic")
    return res


def Minimum(a: OaMatrix, b: OaMatrix) -> OaMatrix:
    """Elementwise minimum with the gradient routed to the smaller operand (ties go to `a`)."""
    ta, tb = F._c(a.Tensor()), F._c(b.Tensor())
    out = OaMatrix(torch.minimum(ta, tb))
    pick = ta <= tb

    def back(g):
        z = torch.zeros_like(g)
        return (torch.where(pick, g, z), torch.where(pick, z, g))

    return AG.attach("Minimum", out, [a, b], back)


def SacActor(q1, q2, log_probability, entropy_coefficient: float = 0.2) -> Optional[OaMatrix]:
    B = q1.Tensor().shape[0] if q1.Tensor().dim() == 1 else 0
    if B <= 0 or not all(_is_f32(m, (B,)) for m in (q1, q2, log_probability)) or not math.isfinite(entropy_coefficient) or entropy_coefficient < 0:
        return None
    L._set("sac_actor")
    return F.Mean(F.Sub(F.Scale(log_probability, entropy_coefficient), Minimum(q1, q2)))
