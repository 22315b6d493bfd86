// Reinforcement-learning support kernels: vector CartPole environment, generalised advantage estimation, fused rollout /
// replay storage, categorical sampling, and the target / clip kernels of the PPO, DQN and SAC losses.
// Behavioural contract: Source/Private/Oa/Ml/Rl/Shader/Compute/{Environment,Gae,Loss,Replay,Rollout}/*.slang of the
// reference.  Every kernel is one thread per environment (or per element); there is no cross-lane state, so results do
// not depend on the launch shape.  All tensors are fp32 / int32 / uint8 and device resident: nothing here reads back.
#include "common.cuh"
#include "api.h"

namespace oa {

__device__ __forceinline__ unsigned rl_mix32(unsigned v) {
  v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu; v ^= v >> 16;
  return v;
}

// uniform in [-0.05, 0.05) from (seed, environment, episode, component); the high 24 bits map exactly onto [0, 1)
__device__ __forceinline__ float cartpole_initial(unsigned seed_lo, unsigned seed_hi, unsigned env, unsigned episode, unsigned comp) {
  unsigned v = rl_mix32(seed_lo ^ rl_mix32(seed_hi + 0x9e3779b9u));
  v = rl_mix32(v ^ rl_mix32(env + 0x85ebca6bu));
  v = rl_mix32(v ^ rl_mix32(episode + 0xc2b2ae35u));
  v = rl_mix32(v ^ rl_mix32(comp + 0x27d4eb2fu));
  return (float)(v >> 8) * (1.0f / 16777216.0f) * 0.1f - 0.05f;
}

__global__ void cartpole_reset_kernel(float* __restrict__ state, unsigned char* __restrict__ done, unsigned* __restrict__ steps,
                                      unsigned* __restrict__ episode, int envs, unsigned seed_lo, unsigned seed_hi, int only_done) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= envs) return;
  if (only_done && done[e] == 0) return;
  const unsigned ep = only_done ? episode[e] + 1u : 0u;
  episode[e] = ep;
  steps[e] = 0u;
  done[e] = 0;
  float4 s;
  s.x = cartpole_initial(seed_lo, seed_hi, e, ep, 0);
  s.y = cartpole_initial(seed_lo, seed_hi, e, ep, 1);
  s.z = cartpole_initial(seed_lo, seed_hi, e, ep, 2);
  s.w = cartpole_initial(seed_lo, seed_hi, e, ep, 3);
  reinterpret_cast<float4*>(state)[e] = s;
}

struct CartPoleParams {
  float gravity, cart_mass, pole_mass, half_len, force, dt, x_limit, angle_limit;
  unsigned max_steps;
};

// Lanes that are already done emit a zero reward and clear flags until they are reset; live lanes keep the pre-action
// observation in `trans_obs`, then advance the state in place with the explicit Euler step of Gymnasium's CartPole-v1.
__global__ void cartpole_step_kernel(const int* __restrict__ action, float* __restrict__ state, float* __restrict__ trans_obs,
                                     float* __restrict__ reward, unsigned char* __restrict__ terminated,
                                     unsigned char* __restrict__ truncated, unsigned char* __restrict__ done,
                                     unsigned* __restrict__ steps, int envs, CartPoleParams p) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= envs) return;
  if (done[e] != 0) {
    reward[e] = 0.f; terminated[e] = 0; truncated[e] = 0;
    return;
  }
  float4 s = reinterpret_cast<float4*>(state)[e];
  reinterpret_cast<float4*>(trans_obs)[e] = s;
  float x = s.x, xv = s.y, th = s.z, thv = s.w;
  const int a = action[e];
  const bool valid = a == 0 || a == 1;
  const float force = a == 1 ? p.force : -p.force;
  const float total = p.cart_mass + p.pole_mass, pml = p.pole_mass * p.half_len;
  const float c = cosf(th), sn = sinf(th);
  const float tmp = (force + pml * thv * thv * sn) / total;
  const float tha = (p.gravity * sn - c * tmp) / (p.half_len * (4.0f / 3.0f - p.pole_mass * c * c / total));
  const float xa = tmp - pml * tha * c / total;
  x += p.dt * xv; xv += p.dt * xa; th += p.dt * thv; thv += p.dt * tha;
  reinterpret_cast<float4*>(state)[e] = make_float4(x, xv, th, thv);
  const unsigned n = steps[e] + 1u;
  steps[e] = n;
  const bool bad = x != x || xv != xv || th != th || thv != thv;
  const bool term = !valid || bad || fabsf(x) > p.x_limit || fabsf(th) > p.angle_limit;
  const bool trunc = !term && n >= p.max_steps;
  reward[e] = valid ? 1.f : 0.f;
  terminated[e] = term; truncated[e] = trunc; done[e] = term || trunc;
}

// Reverse scan over time per environment.  Termination removes the bootstrap value; termination and truncation both cut
// the advantage trace so auto-reset episodes do not leak into each other.
__global__ void gae_kernel(const float* __restrict__ reward, const float* __restrict__ value, const float* __restrict__ next_value,
                           const unsigned char* __restrict__ terminated, const unsigned char* __restrict__ truncated,
                           float* __restrict__ adv, float* __restrict__ ret, int T, int E, float gamma, float lambda) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  float next = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const long long i = (long long)t * E + e;
    const bool term = terminated[i] != 0, trunc = truncated[i] != 0;
    const float v = value[i];
    const float delta = reward[i] + gamma * (term ? 0.f : 1.f) * next_value[i] - v;
    const float a = delta + gamma * lambda * ((term || trunc) ? 0.f : 1.f) * next;
    adv[i] = a; ret[i] = a + v;
    next = a;
  }
}

struct RolloutAppend {
  const float* obs; const int* action; const float* reward; const float* value; const float* next_value; const float* logp;
  const unsigned char* term; const unsigned char* trunc;
  float* o_obs; int* o_action; float* o_reward; float* o_value; float* o_next_value; float* o_logp;
  unsigned char* o_term; unsigned char* o_trunc; unsigned char* o_valid;
  int envs, obs_elems; long long slot;
};

// One launch stores a whole vector transition at time slot `slot` of the time-major rollout.
__global__ void rollout_append_kernel(RolloutAppend a) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long n_obs = (long long)a.envs * a.obs_elems;
  if (i < n_obs) a.o_obs[a.slot * n_obs + i] = a.obs[i];
  if (i < a.envs) {
    const long long o = a.slot * a.envs + i;
    a.o_action[o] = a.action[i]; a.o_reward[o] = a.reward[i]; a.o_value[o] = a.value[i];
    a.o_next_value[o] = a.next_value[i]; a.o_logp[o] = a.logp[i];
    a.o_term[o] = a.term[i]; a.o_trunc[o] = a.trunc[i]; a.o_valid[o] = 1;
  }
}

struct ReplayIo {
  const unsigned* obs; const unsigned* action; const unsigned* next_obs; const float* reward;
  const unsigned char* term; const unsigned char* trunc;
  unsigned* o_obs; unsigned* o_action; unsigned* o_next_obs; float* o_reward; unsigned char* o_term; unsigned char* o_trunc;
  int* o_index;
  unsigned rows, obs_elems, act_elems, capacity, cursor, size, seed_lo, seed_hi;
};

// Ring append of `rows` transitions starting at `cursor` (wraps).  Observations and actions move as 32-bit words, so the
// same kernel serves int32 and fp32 actions.
__global__ void replay_append_kernel(ReplayIo r) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < r.rows * r.obs_elems) {
    const unsigned lane = i / r.obs_elems, c = i - lane * r.obs_elems;
    const unsigned dst = ((r.cursor + lane) % r.capacity) * r.obs_elems + c;
    r.o_obs[dst] = r.obs[i]; r.o_next_obs[dst] = r.next_obs[i];
  }
  if (i < r.rows * r.act_elems) {
    const unsigned lane = i / r.act_elems, c = i - lane * r.act_elems;
    r.o_action[((r.cursor + lane) % r.capacity) * r.act_elems + c] = r.action[i];
  }
  if (i < r.rows) {
    const unsigned dst = (r.cursor + i) % r.capacity;
    r.o_reward[dst] = r.reward[i]; r.o_term[dst] = r.term[i]; r.o_trunc[dst] = r.trunc[i];
  }
}

__device__ __forceinline__ unsigned replay_source(const ReplayIo& r, unsigned lane) {
  return rl_mix32(r.seed_lo ^ rl_mix32(r.seed_hi + lane * 0x9e3779b9u)) % r.size;
}

// Deterministic uniform sampling with replacement: lane -> hash(seed, lane) mod size.
__global__ void replay_sample_kernel(ReplayIo r) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < r.rows * r.obs_elems) {
    const unsigned lane = i / r.obs_elems, c = i - lane * r.obs_elems;
    const unsigned src = replay_source(r, lane) * r.obs_elems + c;
    r.o_obs[i] = r.obs[src]; r.o_next_obs[i] = r.next_obs[src];
  }
  if (i < r.rows * r.act_elems) {
    const unsigned lane = i / r.act_elems, c = i - lane * r.act_elems;
    r.o_action[i] = r.action[replay_source(r, lane) * r.act_elems + c];
  }
  if (i < r.rows) {
    const unsigned src = replay_source(r, i);
    r.o_reward[i] = r.reward[src]; r.o_term[i] = r.term[src]; r.o_trunc[i] = r.trunc[src]; r.o_index[i] = (int)src;
  }
}

// mode 0: per-sample -min(ratio A, clip(ratio) A); mode 1: its gradient w.r.t. the new log-probability of the mean loss
__global__ void ppo_clip_kernel(const float* __restrict__ new_lp, const float* __restrict__ old_lp, const float* __restrict__ adv,
                                float* __restrict__ out, int n, float eps, int mode) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float ratio = expf(new_lp[i] - old_lp[i]), a = adv[i];
  if (mode == 0) {
    const float clipped = fminf(fmaxf(ratio, 1.f - eps), 1.f + eps);
    out[i] = -fminf(ratio * a, clipped * a);
  } else {
    const bool active = (a >= 0.f && ratio > 1.f + eps) || (a < 0.f && ratio < 1.f - eps);
    out[i] = active ? 0.f : -(a * ratio) / (float)n;
  }
}

// reward + discount * max_a nextQ unless terminated (truncation keeps the bootstrap)
__global__ void dqn_target_kernel(const float* __restrict__ reward, const float* __restrict__ next_q,
                                  const unsigned char* __restrict__ terminated, float* __restrict__ out, int batch, int actions,
                                  float discount) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= batch) return;
  float best = -3.402823466e+38f;
  for (int a = 0; a < actions; ++a) best = fmaxf(best, next_q[(long long)r * actions + a]);
  out[r] = reward[r] + (terminated[r] ? 0.f : discount * best);
}

__global__ void sac_target_kernel(const float* __restrict__ reward, const float* __restrict__ q1, const float* __restrict__ q2,
                                  const float* __restrict__ logp, const unsigned char* __restrict__ terminated,
                                  float* __restrict__ out, int batch, float discount, float alpha) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  const float boot = fminf(q1[i], q2[i]) - alpha * logp[i];
  out[i] = reward[i] + (terminated[i] ? 0.f : discount * boot);
}

// Inverse-CDF sample of softmax(logits / temperature) per row; u comes from a counter hash of (seed, row).
// greedy != 0 returns the arg-max instead.
__global__ void sample_categorical_kernel(const float* __restrict__ logits, int* __restrict__ action, int rows, int actions,
                                          float inv_temperature, unsigned seed_lo, unsigned seed_hi, int greedy) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float* l = logits + (long long)r * actions;
  float mx = -3.402823466e+38f;
  int arg = 0;
  for (int a = 0; a < actions; ++a) {
    const float v = l[a] * inv_temperature;
    if (v > mx) { mx = v; arg = a; }
  }
  if (greedy) { action[r] = arg; return; }
  float total = 0.f;
  for (int a = 0; a < actions; ++a) total += expf(l[a] * inv_temperature - mx);
  const unsigned h = rl_mix32(seed_lo ^ rl_mix32(seed_hi + (unsigned)r * 0x9e3779b9u));
  const float u = (float)(h >> 8) * (1.0f / 16777216.0f) * total;
  float acc = 0.f;
  int pick = actions - 1;
  for (int a = 0; a < actions; ++a) {
    acc += expf(l[a] * inv_temperature - mx);
    if (u < acc) { pick = a; break; }
  }
  action[r] = pick;
}

inline int grid1(long long n, int block = 256) { return (int)((n + block - 1) / block); }
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH; }

}  // namespace oa

using namespace oa;

extern "C" {

int oa_rl_cartpole_reset(void* state, void* done, void* steps, void* episode, int envs, unsigned seed_lo, unsigned seed_hi,
                         int only_done, void* stream) {
  if (envs <= 0) return OA_ERR_ARG;
  cartpole_reset_kernel<<<grid1(envs), 256, 0, (cudaStream_t)stream>>>((float*)state, (unsigned char*)done, (unsigned*)steps,
                                                                       (unsigned*)episode, envs, seed_lo, seed_hi, only_done);
  return launch_status();
}

int oa_rl_cartpole_step(const void* action, void* state, void* trans_obs, void* reward, void* terminated, void* truncated,
                        void* done, void* steps, int envs, int max_steps, float gravity, float cart_mass, float pole_mass,
                        float half_len, float force, float dt, float x_limit, float angle_limit, void* stream) {
  if (envs <= 0 || max_steps <= 0) return OA_ERR_ARG;
  CartPoleParams p{gravity, cart_mass, pole_mass, half_len, force, dt, x_limit, angle_limit, (unsigned)max_steps};
  cartpole_step_kernel<<<grid1(envs), 256, 0, (cudaStream_t)stream>>>((const int*)action, (float*)state, (float*)trans_obs,
                                                                      (float*)reward, (unsigned char*)terminated,
                                                                      (unsigned char*)truncated, (unsigned char*)done,
                                                                      (unsigned*)steps, envs, p);
  return launch_status();
}

int oa_rl_gae(const void* reward, const void* value, const void* next_value, const void* terminated, const void* truncated,
              void* adv, void* ret, int T, int E, float gamma, float lambda, void* stream) {
  if (T <= 0 || E <= 0) return OA_ERR_ARG;
  gae_kernel<<<grid1(E, 64), 64, 0, (cudaStream_t)stream>>>((const float*)reward, (const float*)value, (const float*)next_value,
                                                            (const unsigned char*)terminated, (const unsigned char*)truncated,
                                                            (float*)adv, (float*)ret, T, E, gamma, lambda);
  return launch_status();
}

int oa_rl_rollout_append(const void* obs, const void* action, const void* reward, const void* value, const void* next_value,
                         const void* logp, const void* term, const void* trunc, void* o_obs, void* o_action, void* o_reward,
                         void* o_value, void* o_next_value, void* o_logp, void* o_term, void* o_trunc, void* o_valid, int envs,
                         int obs_elems, int slot, void* stream) {
  if (envs <= 0 || obs_elems <= 0 || slot < 0) return OA_ERR_ARG;
  RolloutAppend a{(const float*)obs, (const int*)action, (const float*)reward, (const float*)value, (const float*)next_value,
                  (const float*)logp, (const unsigned char*)term, (const unsigned char*)trunc, (float*)o_obs, (int*)o_action,
                  (float*)o_reward, (float*)o_value, (float*)o_next_value, (float*)o_logp, (unsigned char*)o_term,
                  (unsigned char*)o_trunc, (unsigned char*)o_valid, envs, obs_elems, slot};
  rollout_append_kernel<<<grid1((long long)envs * obs_elems), 256, 0, (cudaStream_t)stream>>>(a);
  return launch_status();
}

// mode 0: append `rows` transitions at `cursor` of a ring with `capacity` rows; mode 1: sample `rows` rows out of the first
// `size` stored rows into the o_* batch tensors (o_index receives the source rows).
int oa_rl_replay(int mode, const void* obs, const void* action, const void* next_obs, const void* reward, const void* term,
                 const void* trunc, void* o_obs, void* o_action, void* o_next_obs, void* o_reward, void* o_term, void* o_trunc,
                 void* o_index, int rows, int obs_elems, int act_elems, int capacity, int cursor, int size, unsigned seed_lo,
                 unsigned seed_hi, void* stream) {
  if (rows <= 0 || obs_elems <= 0 || act_elems <= 0 || capacity <= 0) return OA_ERR_ARG;
  if (mode == 1 && (size <= 0 || !o_index)) return OA_ERR_ARG;
  if (mode == 0 && rows > capacity) return OA_ERR_ARG;
  ReplayIo r{(const unsigned*)obs, (const unsigned*)action, (const unsigned*)next_obs, (const float*)reward,
             (const unsigned char*)term, (const unsigned char*)trunc, (unsigned*)o_obs, (unsigned*)o_action, (unsigned*)o_next_obs,
             (float*)o_reward, (unsigned char*)o_term, (unsigned char*)o_trunc, (int*)o_index, (unsigned)rows, (unsigned)obs_elems,
             (unsigned)act_elems, (unsigned)capacity, (unsigned)cursor, (unsigned)size, seed_lo, seed_hi};
  const long long n = (long long)rows * (obs_elems > act_elems ? obs_elems : act_elems);
  if (mode == 0) replay_append_kernel<<<grid1(n), 256, 0, (cudaStream_t)stream>>>(r);
  else replay_sample_kernel<<<grid1(n), 256, 0, (cudaStream_t)stream>>>(r);
  return launch_status();
}

int oa_rl_ppo_clip(const void* new_lp, const void* old_lp, const void* adv, void* out, int n, float eps, int backward,
                   void* stream) {
  if (n <= 0) return OA_ERR_ARG;
  ppo_clip_kernel<<<grid1(n), 256, 0, (cudaStream_t)stream>>>((const float*)new_lp, (const float*)old_lp, (const float*)adv,
                                                              (float*)out, n, eps, backward);
  return launch_status();
}

int oa_rl_dqn_target(const void* reward, const void* next_q, const void* terminated, void* out, int batch, int actions,
                     float discount, void* stream) {
  if (batch <= 0 || actions <= 0) return OA_ERR_ARG;
  dqn_target_kernel<<<grid1(batch), 256, 0, (cudaStream_t)stream>>>((const float*)reward, (const float*)next_q,
                                                                    (const unsigned char*)terminated, (float*)out, batch, actions,
                                                                    discount);
  return launch_status();
}

int oa_rl_sac_target(const void* reward, const void* q1, const void* q2, const void* logp, const void* terminated, void* out,
                     int batch, float discount, float alpha, void* stream) {
  if (batch <= 0) return OA_ERR_ARG;
  sac_target_kernel<<<grid1(batch), 256, 0, (cudaStream_t)stream>>>((const float*)reward, (const float*)q1, (const float*)q2,
                                                                    (const float*)logp, (const unsigned char*)terminated,
                                                                    (float*)out, batch, discount, alpha);
  return launch_status();
}

int oa_rl_sample_categorical(const void* logits, void* action, int rows, int actions, float temperature, unsigned seed_lo,
                             unsigned seed_hi, int greedy, void* stream) {
  if (rows <= 0 || actions <= 0 || !(temperature > 0.f)) return OA_ERR_ARG;
  sample_categorical_kernel<<<grid1(rows), 256, 0, (cudaStream_t)stream>>>((const float*)logits, (int*)action, rows, actions,
                                                                          1.0f / temperature, seed_lo, seed_hi, greedy);
  return launch_status();
}

}  // extern "C"
