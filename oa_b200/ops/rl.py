"""Raw-tensor reinforcement-learning ops: CUDA tensors run csrc/kernels/rl.cu, CPU tensors run the same arithmetic in
PyTorch (the oracle of the GPU tests; hashes are evaluated bit-exactly so both paths draw the same samples).

Contract of every op: Source/Private/Oa/Ml/Rl/Shader/Compute/*/*.slang of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N
from . import kernels as K

M32 = 0xFFFFFFFF


def _mix32(v: torch.Tensor) -> torch.Tensor:
    """The 32-bit finaliser of rl.cu on int64 lanes (values kept in [0, 2^32))."""
    v = v & M32
    v = v ^ (v >> 16)
    v = (v * 0x7FEB352D) & M32
    v = v ^ (v >> 15)
    v = (v * 0x846CA68B) & M32
    v = v ^ (v >> 16)
    return v


def _split(seed: int):
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    return seed & M32, seed >> 32


def _lane_hash(seed: int, lanes: torch.Tensor) -> torch.Tensor:
    lo, hi = _split(seed)
    return _mix32(lo ^ _mix32((hi + lanes.to(torch.int64) * 0x9E3779B9) & M32))


@dataclass
class CartPoleParams:
    gravity: float = 9.8
    cart_mass: float = 1.0
    pole_mass: float = 0.1
    half_len: float = 0.5
    force: float = 10.0
    dt: float = 0.02
    x_limit: float = 2.4
    angle_limit: float = 0.2094395102
    max_steps: int = 500


def cartpole_reset(state, done, steps, episode, seed: int, only_done: bool) -> None:
    """state [E, 4] fp32, done [E] uint8, steps / episode [E] int32 - all updated in place."""
    E = state.shape[0]
    lo, hi = _split(seed)
    if state.is_cuda:
        lib = N.require()
        K._launch(lib.oa_rl_cartpole_reset(state.data_ptr(), done.data_ptr(), steps.data_ptr(), episode.data_ptr(), E, lo, hi,
                                           int(only_done), N.stream()), "oa_rl_cartpole_reset")
        return
    sel = done.ne(0) if only_done else torch.ones(E, dtype=torch.bool)
    ep = torch.where(sel, episode.to(torch.int64) + 1 if only_done else torch.zeros(E, dtype=torch.int64), episode.to(torch.int64))
    env = torch.arange(E, dtype=torch.int64)
    base = _mix32(torch.tensor(lo, dtype=torch.int64) ^ _mix32(torch.tensor((hi + 0x9E3779B9) & M32, dtype=torch.int64)))
    v = _mix32(base ^ _mix32((env + 0x85EBCA6B) & M32))
    v = _mix32(v ^ _mix32((ep + 0xC2B2AE35) & M32))
    cols = []
    for c in range(4):
        h = _mix32(v ^ _mix32(torch.tensor((c + 0x27D4EB2F) & M32, dtype=torch.int64)))
        cols.append((h >> 8).to(torch.float32) * (1.0 / 16777216.0) * 0.1 - 0.05)
    new = torch.stack(cols, 1)
    state[sel] = new[sel]
    episode[sel] = ep[sel].to(episode.dtype)
    steps[sel] = 0
    done[sel] = 0


def cartpole_step(action, state, trans_obs, reward, terminated, truncated, done, steps, p: CartPoleParams) -> None:
    E = state.shape[0]
    if state.is_cuda:
        lib = N.require()
        K._launch(lib.oa_rl_cartpole_step(action.data_ptr(), state.data_ptr(), trans_obs.data_ptr(), reward.data_ptr(),
                                          terminated.data_ptr(), truncated.data_ptr(), done.data_ptr(), steps.data_ptr(), E,
                                          int(p.max_steps), p.gravity, p.cart_mass, p.pole_mass, p.half_len, p.force, p.dt,
                                          p.x_limit, p.angle_limit, N.stream()), "oa_rl_cartpole_step")
        return
    live = done.eq(0)
    reward[~live] = 0.0
    terminated[~live] = 0
    truncated[~live] = 0
    trans_obs[live] = state[live]
    f32 = lambda v: torch.tensor(v, dtype=torch.float32)
    x, xv, th, thv = state.unbind(1)
    valid = (action == 0) | (action == 1)
    force = torch.where(action == 1, f32(p.force), f32(-p.force))
    total, pml = f32(p.cart_mass) + f32(p.pole_mass), f32(p.pole_mass) * f32(p.half_len)
    c, sn = torch.cos(th), torch.sin(th)
    tmp = (force + pml * thv * thv * sn) / total
    tha = (f32(p.gravity) * sn - c * tmp) / (f32(p.half_len) * (f32(4.0) / f32(3.0) - f32(p.pole_mass) * c * c / total))
    xa = tmp - pml * tha * c / total
    dt = f32(p.dt)
    nx, nxv, nth, nthv = x + dt * xv, xv + dt * xa, th + dt * thv, thv + dt * tha
    new = torch.stack((nx, nxv, nth, nthv), 1)
    n = steps + 1
    bad = torch.isnan(new).any(1)
    term = ~valid | bad | (nx.abs() > p.x_limit) | (nth.abs() > p.angle_limit)
    trunc = ~term & (n >= p.max_steps)
    state[live] = new[live]
    steps[live] = n[live]
    reward[live] = valid[live].float()
    terminated[live] = term[live].to(terminated.dtype)
    truncated[live] = trunc[live].to(truncated.dtype)
    done[live] = (term | trunc)[live].to(done.dtype)


def gae(reward, value, next_value, terminated, truncated, adv, ret, gamma: float, lam: float) -> None:
    """[T, E] fp32 / uint8 inputs -> adv, ret [T, E] written in place."""
    T, E = reward.shape
    if reward.is_cuda:
        lib = N.require()
        K._launch(lib.oa_rl_gae(reward.data_ptr(), value.data_ptr(), next_value.data_ptr(), terminated.data_ptr(),
                                truncated.data_ptr(), adv.data_ptr(), ret.data_ptr(), T, E, float(gamma), float(lam), N.stream()),
                  "oa_rl_gae")
        return
    nxt = torch.zeros(E)
    for t in range(T - 1, -1, -1):
        term, trunc = terminated[t].ne(0), truncated[t].ne(0)
        delta = reward[t] + gamma * (~term).float() * next_value[t] - value[t]
        a = delta + gamma * lam * (~(term | trunc)).float() * nxt
        adv[t] = a
        ret[t] = a + value[t]
        nxt = a


def rollout_append(src: dict, dst: dict, slot: int) -> None:
    """src: obs [E, ...], action int32 [E], reward, value, next_value, logp fp32 [E], term, trunc uint8 [E];
    dst: the [T, E, ...] tensors of the same names plus `valid`."""
    E = src["action"].shape[0]
    obs_elems = src["obs"].numel() // E
    if src["obs"].is_cuda:
        lib = N.require()
        p = lambda d, k: d[k].data_ptr()
        K._launch(lib.oa_rl_rollout_append(p(src, "obs"), p(src, "action"), p(src, "reward"), p(src, "value"), p(src, "next_value"),
                                           p(src, "logp"), p(src, "term"), p(src, "trunc"), p(dst, "obs"), p(dst, "action"),
                                           p(dst, "reward"), p(dst, "value"), p(dst, "next_value"), p(dst, "logp"), p(dst, "term"),
                                           p(dst, "trunc"), p(dst, "valid"), E, obs_elems, int(slot), N.stream()),
                  "oa_rl_rollout_append")
        return
    for k in ("obs", "action", "reward", "value", "next_value", "logp", "term", "trunc"):
        dst[k][slot] = src[k].reshape(dst[k][slot].shape)
    dst["valid"][slot] = 1


_REPLAY_KEYS = ("obs", "action", "next_obs", "reward", "term", "trunc")


def replay_append(src: dict, store: dict, cursor: int, capacity: int) -> None:
    rows = src["reward"].shape[0]
    obs_e, act_e = src["obs"].numel() // rows, src["action"].numel() // rows
    if src["obs"].is_cuda:
        lib = N.require()
        p = lambda d, k: d[k].data_ptr()
        K._launch(lib.oa_rl_replay(0, *[p(src, k) for k in _REPLAY_KEYS], *[p(store, k) for k in _REPLAY_KEYS], None, rows, obs_e,
                                   act_e, capacity, cursor, 0, 0, 0, N.stream()), "oa_rl_replay_append")
        return
    idx = (cursor + torch.arange(rows)) % capacity
    for k in _REPLAY_KEYS:
        store[k][idx] = src[k].reshape(rows, *store[k].shape[1:])


def replay_sample(store: dict, out: dict, size: int, seed: int) -> None:
    """out: batch tensors of the stored names plus `index` int32 [batch]."""
    rows = out["reward"].shape[0]
    obs_e, act_e = out["obs"].numel() // rows, out["action"].numel() // rows
    lo, hi = _split(seed)
    if out["obs"].is_cuda:
        lib = N.require()
        p = lambda d, k: d[k].data_ptr()
        K._launch(lib.oa_rl_replay(1, *[p(store, k) for k in _REPLAY_KEYS], *[p(out, k) for k in _REPLAY_KEYS], p(out, "index"), rows,
                                   obs_e, act_e, store["reward"].shape[0], 0, int(size), lo, hi, N.stream()), "oa_rl_replay_sample")
        return
    src = (_lane_hash(seed, torch.arange(rows)) % size).long()
    for k in _REPLAY_KEYS:
        out[k].copy_(store[k][src])
    out["index"].copy_(src.to(torch.int32))


def ppo_clip(new_lp, old_lp, adv, eps: float, backward: bool) -> torch.Tensor:
    n = new_lp.numel()
    if new_lp.is_cuda:
        out = torch.empty_like(new_lp)
        lib = N.require()
        K._launch(lib.oa_rl_ppo_clip(new_lp.data_ptr(), old_lp.data_ptr(), adv.data_ptr(), out.data_ptr(), n, float(eps), int(backward),
                                     N.stream()), "oa_rl_ppo_clip")
        return out
    ratio = torch.exp(new_lp - old_lp)
    if not backward:
        return -torch.minimum(ratio * adv, ratio.clamp(1 - eps, 1 + eps) * adv)
    active = ((adv >= 0) & (ratio > 1 + eps)) | ((adv < 0) & (ratio < 1 - eps))
    return torch.where(active, torch.zeros_like(adv), -(adv * ratio) / n)


def dqn_target(reward, next_q, terminated, discount: float) -> torch.Tensor:
    B, A = next_q.shape
    if reward.is_cuda:
        out = torch.empty_like(reward)
        lib = N.require()
        K._launch(lib.oa_rl_dqn_target(reward.data_ptr(), next_q.data_ptr(), terminated.data_ptr(), out.data_ptr(), B, A, float(discount),
                                       N.stream()), "oa_rl_dqn_target")
        return out
    return reward + torch.where(terminated.ne(0), torch.zeros_like(reward), discount * next_q.max(1).values)


def sac_target(reward, q1, q2, logp, terminated, discount: float, alpha: float) -> torch.Tensor:
    if reward.is_cuda:
        out = torch.empty_like(reward)
        lib = N.require()
        K._launch(lib.oa_rl_sac_target(reward.data_ptr(), q1.data_ptr(), q2.data_ptr(), logp.data_ptr(), terminated.data_ptr(),
                                       out.data_ptr(), reward.numel(), float(discount), float(alpha), N.stream()), "oa_rl_sac_target")
        return out
    boot = torch.minimum(q1, q2) - alpha * logp
    return reward + torch.where(terminated.ne(0), torch.zeros_like(reward), discount * boot)


def sample_categorical(logits, seed: int, temperature: float = 1.0, greedy: bool = False) -> torch.Tensor:
    """logits fp32 [rows, actions] -> int32 [rows]: inverse-CDF draw from softmax(logits / temperature) with
    u = hash(seed, row) / 2^24, or the arg-max when greedy."""
    rows, A = logits.shape
    lo, hi = _split(seed)
    if logits.is_cuda:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        lib = N.require()
        K._launch(lib.oa_rl_sample_categorical(logits.data_ptr(), out.data_ptr(), rows, A, float(temperature), lo, hi, int(greedy),
                                               N.stream()), "oa_rl_sample_categorical")
        return out
    v = logits * (1.0 / temperature)
    if greedy:
        return v.argmax(1).to(torch.int32)
    e = torch.exp(v - v.max(1, keepdim=True).values)
    u = (_lane_hash(seed, torch.arange(rows)) >> 8).to(torch.float32) * (1.0 / 16777216.0) * e.sum(1)
    acc = torch.cumsum(e, 1)
    return (acc <= u[:, None]).sum(1).clamp(max=A - 1).to(torch.int32)
