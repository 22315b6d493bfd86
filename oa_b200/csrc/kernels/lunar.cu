// LunarLander3d: batched rigid-body lander over a height-field terrain, one thread per lane.
//
// Contract: Source/Private/Oa/Ml/Rl/Shader/Compute/Environment/RlLunarLander3dStep.slang (config indices :3-58, state
// layout :60-82, end reasons :84-92, observation :563-632, step :658-867) and RlLunarLander3dReset.slang.  Each lane
// integrates `substeps` semi-implicit Euler steps (main engine along the body's up axis, attitude torque with the
// gyroscopic term, quaternion stored scalar-first), resolves three hull spheres and four feet against the
// triangulated height field with sequential impulses, and then scores the step.  Lanes never interact, so there is
// no synchronisation and the result does not depend on the launch shape.  The whole state of a lane (32 floats,
// 16 integers) lives in registers for the duration of the step; the terrain (a few KB) is served by L1 / L2.
#include "common.cuh"
#include "api.h"

namespace oa {

namespace lunar {

enum : int {
  C_DT = 0, C_GRAVITY, C_MASS, C_IX, C_IY, C_IZ, C_THRUST, C_TORQUE, C_FUEL_CAP, C_MAIN_RATE, C_ATT_RATE, C_RESTITUTION, C_FRICTION,
  C_SLOP, C_CORR_FRAC, C_MAX_CORR, C_MAX_IMPULSE, C_MAX_BIAS, C_MIN_Y, C_MAX_Y, C_SAFE_LIN, C_SAFE_ANG, C_SAFE_TILT, C_HARD_FOOT,
  C_POS_SCALE, C_VEL_SCALE, C_ANG_SCALE, C_TERRAIN_SCALE, C_FOOT_SCALE, C_PROBE, C_GAMMA, C_W_POS, C_W_VEL, C_W_TILT, C_W_ANG,
  C_W_MAIN_FUEL, C_W_ATT_FUEL, C_R_SOFT, C_R_DWELL, C_R_SUCCESS, C_R_FAIL, C_CELL, C_MIN_X, C_MAX_X, C_MIN_Z, C_MAX_Z, C_PAD, C_SUPPORT,
  C_TERRAIN_TOP = C_SUPPORT + 28,   // no terrain vertex lies above this height
  C_REACH,                          // largest |support offset| + radius: no support sphere reaches further from the centre
  C_COUNT
};
enum : int { N_SUBSTEPS = 0, N_ITERATIONS, N_DWELL, N_MAX_STEPS, N_CELLS_X, N_CELLS_Z };
enum : int { S_POS = 0, S_VEL = 3, S_QUAT = 6, S_ANG = 10, S_FUEL = 13, S_THROTTLE = 14, S_ATT = 15, S_BODY_IMP = 18, S_FOOT_IMP = 21, S_RETURN = 25 };
enum : int { U_ACTION = 0, U_BODY, U_FOOT, U_PAD, U_REWARDED, U_STEP, U_DWELL, U_TERM, U_TRUNC, U_REASON, U_EPISODE };
enum : int { END_SAFE = 1, END_BODY = 2, END_HARD_FOOT = 3, END_OOB = 4, END_NUMERIC = 5, END_TIME = 6, END_STOP = 7, END_BAD_ACTION = 8 };

struct Config { float f[C_COUNT]; int n[6]; };

struct V3 { float x, y, z; };
__device__ __forceinline__ V3 v3(float x, float y, float z) { return V3{x, y, z}; }
__device__ __forceinline__ V3 operator+(V3 a, V3 b) { return v3(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ V3 operator-(V3 a, V3 b) { return v3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ V3 operator*(V3 a, float s) { return v3(a.x * s, a.y * s, a.z * s); }
__device__ __forceinline__ V3 operator*(V3 a, V3 b) { return v3(a.x * b.x, a.y * b.y, a.z * b.z); }
__device__ __forceinline__ V3 operator/(V3 a, float s) { return v3(a.x / s, a.y / s, a.z / s); }
__device__ __forceinline__ float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ V3 cross(V3 a, V3 b) { return v3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
__device__ __forceinline__ float length(V3 a) { return sqrtf(dot(a, a)); }
__device__ __forceinline__ bool finite3(V3 a) { return isfinite(a.x) && isfinite(a.y) && isfinite(a.z); }

struct Quat { float w, x, y, z; };
// v' = v + w t + u x t with t = 2 u x v (u = vector part, negated for the inverse rotation)
__device__ __forceinline__ V3 rotate(Quat q, V3 v, bool inverse = false) {
  const V3 u = inverse ? v3(-q.x, -q.y, -q.z) : v3(q.x, q.y, q.z);
  const V3 t = cross(u, v) * 2.0f;
  return v + t * q.w + cross(u, t);
}

struct Body {
  V3 pos, vel, ang, att;
  Quat q;
  float fuel, throttle, body_imp[3], foot_imp[4], ret;
  int u[16];
};

__device__ __forceinline__ bool finite_body(const Body& b) {
  return finite3(b.pos) && finite3(b.vel) && finite3(b.ang) && isfinite(b.q.w) && isfinite(b.q.x) && isfinite(b.q.y) && isfinite(b.q.z) &&
         isfinite(b.fuel);
}

__device__ void load_body(Body& b, const float* sf, const int* su) {
  b.pos = v3(sf[S_POS], sf[S_POS + 1], sf[S_POS + 2]);
  b.vel = v3(sf[S_VEL], sf[S_VEL + 1], sf[S_VEL + 2]);
  b.q = Quat{sf[S_QUAT], sf[S_QUAT + 1], sf[S_QUAT + 2], sf[S_QUAT + 3]};
  b.ang = v3(sf[S_ANG], sf[S_ANG + 1], sf[S_ANG + 2]);
  b.fuel = sf[S_FUEL]; b.throttle = sf[S_THROTTLE];
  b.att = v3(sf[S_ATT], sf[S_ATT + 1], sf[S_ATT + 2]);
  for (int i = 0; i < 3; ++i) b.body_imp[i] = sf[S_BODY_IMP + i];
  for (int i = 0; i < 4; ++i) b.foot_imp[i] = sf[S_FOOT_IMP + i];
  b.ret = sf[S_RETURN];
  for (int i = 0; i < 16; ++i) b.u[i] = su[i];
}

__device__ void store_body(const Body& b, float* sf, int* su) {
  sf[S_POS] = b.pos.x; sf[S_POS + 1] = b.pos.y; sf[S_POS + 2] = b.pos.z;
  sf[S_VEL] = b.vel.x; sf[S_VEL + 1] = b.vel.y; sf[S_VEL + 2] = b.vel.z;
  sf[S_QUAT] = b.q.w; sf[S_QUAT + 1] = b.q.x; sf[S_QUAT + 2] = b.q.y; sf[S_QUAT + 3] = b.q.z;
  sf[S_ANG] = b.ang.x; sf[S_ANG + 1] = b.ang.y; sf[S_ANG + 2] = b.ang.z;
  sf[S_FUEL] = b.fuel; sf[S_THROTTLE] = b.throttle;
  sf[S_ATT] = b.att.x; sf[S_ATT + 1] = b.att.y; sf[S_ATT + 2] = b.att.z;
  for (int i = 0; i < 3; ++i) sf[S_BODY_IMP + i] = b.body_imp[i];
  for (int i = 0; i < 4; ++i) sf[S_FOOT_IMP + i] = b.foot_imp[i];
  sf[S_RETURN] = b.ret;
  for (int i = 0; i < 16; ++i) su[i] = b.u[i];
}

struct Ground { bool inside; float height; V3 normal; };

// Each cell is split along its (0,0)-(1,1) diagonal; the sample lies on the plane of its triangle.
__device__ Ground ground_at(const Config& c, const float* __restrict__ terrain, float x, float z) {
  Ground g{false, 0.f, v3(0.f, 1.f, 0.f)};
  if (!(x >= c.f[C_MIN_X] && x <= c.f[C_MAX_X] && z >= c.f[C_MIN_Z] && z <= c.f[C_MAX_Z])) return g;
  const int nx = c.n[N_CELLS_X], nz = c.n[N_CELLS_Z];
  const float cell = c.f[C_CELL];
  const float gx = (x - c.f[C_MIN_X]) / cell, gz = (z - c.f[C_MIN_Z]) / cell;
  const bool end_x = gx >= (float)nx, end_z = gz >= (float)nz;
  const int cx = end_x ? nx - 1 : (int)floorf(gx), cz = end_z ? nz - 1 : (int)floorf(gz);
  const float lx = end_x ? 1.f : gx - (float)cx, lz = end_z ? 1.f : gz - (float)cz;
  const int row = nx + 1, i00 = cz * row + cx;
  const float h00 = terrain[i00], h10 = terrain[i00 + 1], h01 = terrain[i00 + row], h11 = terrain[i00 + row + 1];
  float ddx, ddz;
  if (lz <= lx) { g.height = h00 + lx * (h10 - h00) + lz * (h11 - h10); ddx = (h10 - h00) / cell; ddz = (h11 - h10) / cell; }
  else { g.height = h00 + lx * (h11 - h01) + lz * (h01 - h00); ddx = (h11 - h01) / cell; ddz = (h01 - h00) / cell; }
  const V3 n = v3(-ddx, 1.f, -ddz);
  g.normal = n / length(n);
  g.inside = true;
  return g;
}

__device__ __forceinline__ V3 support_offset(const Config& c, int k) { return v3(c.f[C_SUPPORT + 4 * k], c.f[C_SUPPORT + 4 * k + 1], c.f[C_SUPPORT + 4 * k + 2]); }
__device__ __forceinline__ float support_radius(const Config& c, int k) { return c.f[C_SUPPORT + 4 * k + 3]; }
__device__ __forceinline__ V3 inverse_inertia(const Config& c) { return v3(1.0f / c.f[C_IX], 1.0f / c.f[C_IY], 1.0f / c.f[C_IZ]); }

__device__ float effective_inverse_mass(const Config& c, const Body& b, V3 lever, V3 dir) {
  const V3 rb = rotate(b.q, cross(lever, dir), true);
  return 1.0f / c.f[C_MASS] + dot(rb, rb * inverse_inertia(c));
}

__device__ void apply_impulse(const Config& c, Body& b, V3 lever, V3 impulse) {
  b.vel = b.vel + impulse / c.f[C_MASS];
  b.ang = b.ang + rotate(b.q, cross(lever, impulse), true) * inverse_inertia(c);
}

struct Diag { float foot_speed; bool foot_hit, body_hit; };

__device__ void resolve_support(const Config& c, const float* __restrict__ terrain, Body& b, int k, float h, Diag& d) {
  const V3 center = b.pos + rotate(b.q, support_offset(c, k));
  const Ground g = ground_at(c, terrain, center.x, center.z);
  if (!g.inside) return;
  const float sep = center.y - support_radius(c, k) - g.height;
  if (!(sep < 0.f)) return;
  const float pen = -sep;
  const V3 lever = center - b.pos;
  V3 pv = b.vel + cross(rotate(b.q, b.ang), lever);
  const float vn = dot(pv, g.normal);
  const float closing = fmaxf(-vn, 0.f);
  const bool foot = k >= 3;
  if (foot) { d.foot_hit = true; d.foot_speed = fmaxf(d.foot_speed, closing); }
  const float bias = fminf(c.f[C_MAX_BIAS], pen * c.f[C_CORR_FRAC] / h);
  float jn = fmaxf(-(1.0f + c.f[C_RESTITUTION]) * vn + bias, 0.f) / effective_inverse_mass(c, b, lever, g.normal);
  jn = fminf(fmaxf(jn, 0.f), c.f[C_MAX_IMPULSE]);
  apply_impulse(c, b, lever, g.normal * jn);
  pv = b.vel + cross(rotate(b.q, b.ang), lever);
  const V3 tv = pv - g.normal * dot(pv, g.normal);
  const float ts = length(tv);
  if (ts > 1.0e-12f) {
    const V3 tdir = (tv * -1.0f) / ts;
    float jt = fminf(ts / effective_inverse_mass(c, b, lever, tdir), c.f[C_FRICTION] * jn);
    jt = fminf(fmaxf(jt, 0.f), c.f[C_MAX_IMPULSE]);
    apply_impulse(c, b, lever, tdir * jt);
  }
  b.pos = b.pos + g.normal * fminf(c.f[C_MAX_CORR], pen * c.f[C_CORR_FRAC]);
  if (foot) { b.u[U_FOOT] |= 1 << (k - 3); b.foot_imp[k - 3] += jn; }
  else { d.body_hit = true; b.u[U_BODY] |= 1 << k; b.body_imp[k] += jn; }
}

__device__ void refresh_contacts(const Config& c, const float* __restrict__ terrain, Body& b) {
  int body = 0, foot = 0, pad = 0;
  for (int k = 0; k < 7; ++k) {
    const V3 center = b.pos + rotate(b.q, support_offset(c, k));
    const Ground g = ground_at(c, terrain, center.x, center.z);
    const bool touch = g.inside && center.y - support_radius(c, k) - g.height <= c.f[C_SLOP];
    if (k < 3) { if (touch) body |= 1 << k; }
    else {
      if (touch) foot |= 1 << (k - 3);
      if (g.inside && fmaxf(fabsf(center.x), fabsf(center.z)) <= c.f[C_PAD]) pad |= 1 << (k - 3);
    }
  }
  b.u[U_BODY] = body; b.u[U_FOOT] = foot; b.u[U_PAD] = pad;
}

__device__ float potential(const Config& c, const Body& b) {
  if (!finite_body(b)) return 0.f;
  const V3 up = rotate(b.q, v3(0.f, 1.f, 0.f));
  const float cost = c.f[C_W_POS] * fminf(1.f, length(b.pos) / c.f[C_POS_SCALE]) + c.f[C_W_VEL] * fminf(1.f, length(b.vel) / c.f[C_VEL_SCALE]) +
                     c.f[C_W_TILT] * fminf(fmaxf((1.0f - up.y) * 0.5f, 0.f), 1.f) + c.f[C_W_ANG] * fminf(1.f, length(b.ang) / c.f[C_ANG_SCALE]);
  return -cost;
}

__device__ __forceinline__ float unit(float v, float scale) { return fminf(fmaxf(v / scale, -1.f), 1.f); }

__device__ void write_observation(const Config& c, const float* __restrict__ terrain, const Body& b, float* __restrict__ o) {
  if (!finite_body(b)) { for (int i = 0; i < 33; ++i) o[i] = 0.f; return; }
  o[0] = unit(b.pos.x, c.f[C_POS_SCALE]); o[1] = unit(b.pos.y, c.f[C_POS_SCALE]); o[2] = unit(b.pos.z, c.f[C_POS_SCALE]);
  o[3] = unit(b.vel.x, c.f[C_VEL_SCALE]); o[4] = unit(b.vel.y, c.f[C_VEL_SCALE]); o[5] = unit(b.vel.z, c.f[C_VEL_SCALE]);
  const V3 up = rotate(b.q, v3(0.f, 1.f, 0.f)), fwd = rotate(b.q, v3(0.f, 0.f, -1.f));
  o[6] = unit(up.x, 1.f); o[7] = unit(up.y, 1.f); o[8] = unit(up.z, 1.f);
  o[9] = unit(fwd.x, 1.f); o[10] = unit(fwd.y, 1.f); o[11] = unit(fwd.z, 1.f);
  o[12] = unit(b.ang.x, c.f[C_ANG_SCALE]); o[13] = unit(b.ang.y, c.f[C_ANG_SCALE]); o[14] = unit(b.ang.z, c.f[C_ANG_SCALE]);
  int at = 15;
  for (int pz = -1; pz <= 1; ++pz)
    for (int px = -1; px <= 1; ++px) {
      const Ground g = ground_at(c, terrain, b.pos.x + (float)px * c.f[C_PROBE], b.pos.z + (float)pz * c.f[C_PROBE]);
      o[at++] = unit(g.inside ? b.pos.y - g.height : c.f[C_TERRAIN_SCALE], c.f[C_TERRAIN_SCALE]);
    }
  for (int k = 3; k < 7; ++k) {
    const V3 center = b.pos + rotate(b.q, support_offset(c, k));
    const Ground g = ground_at(c, terrain, center.x, center.z);
    o[at++] = unit(g.inside ? center.y - support_radius(c, k) - g.height : c.f[C_FOOT_SCALE], c.f[C_FOOT_SCALE]);
  }
  for (int f = 0; f < 4; ++f) o[at++] = (b.u[U_FOOT] >> f) & 1 ? 1.f : 0.f;
  o[at] = fminf(fmaxf(b.fuel / c.f[C_FUEL_CAP], 0.f), 1.f);
}

}  // namespace lunar

using namespace lunar;

__global__ void __launch_bounds__(128)
lunar_step_kernel(const Config c, const float* __restrict__ terrain, const int* __restrict__ action, const unsigned char* __restrict__ external_stop,
                  float* __restrict__ state_f, int* __restrict__ state_u, float* __restrict__ trans_obs, float* __restrict__ obs,
                  float* __restrict__ reward, unsigned char* __restrict__ terminated, unsigned char* __restrict__ truncated,
                  int* __restrict__ end_reason, int envs) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= envs) return;
  float* sf = state_f + (long long)e * 32;
  int* su = state_u + (long long)e * 16;
  float* o = obs + (long long)e * 33;
  for (int i = 0; i < 33; ++i) trans_obs[(long long)e * 33 + i] = o[i];
  Body b;
  load_body(b, sf, su);
  if (b.u[U_TERM] != 0 || b.u[U_TRUNC] != 0) {          // finished lanes idle until they are reset
    reward[e] = 0.f; terminated[e] = b.u[U_TERM] != 0; truncated[e] = b.u[U_TRUNC] != 0; end_reason[e] = b.u[U_REASON];
    return;
  }
  const int act = action[e];
  if (act < 0 || act >= 8) {
    b.u[U_STEP] += 1; b.u[U_TERM] = 1; b.u[U_REASON] = END_BAD_ACTION;
    b.ret += c.f[C_R_FAIL];
    store_body(b, sf, su);
    write_observation(c, terrain, b, o);
    reward[e] = c.f[C_R_FAIL]; terminated[e] = 1; truncated[e] = 0; end_reason[e] = END_BAD_ACTION;
    return;
  }
  if (external_stop != nullptr && external_stop[e] != 0) {
    b.u[U_TRUNC] = 1; b.u[U_REASON] = END_STOP;
    store_body(b, sf, su);
    write_observation(c, terrain, b, o);
    reward[e] = 0.f; terminated[e] = 0; truncated[e] = 1; end_reason[e] = END_STOP;
    return;
  }
  const float pot_before = potential(c, b);
  b.u[U_ACTION] = act;
  b.throttle = 0.f; b.att = v3(0.f, 0.f, 0.f);
  b.u[U_BODY] = 0; b.u[U_FOOT] = 0; b.u[U_PAD] = 0;
  for (int i = 0; i < 3; ++i) b.body_imp[i] = 0.f;
  for (int i = 0; i < 4; ++i) b.foot_imp[i] = 0.f;
  Diag d{0.f, false, false};
  float main_used = 0.f, att_used = 0.f;
  bool valid = finite_body(b);
  const int substeps = c.n[N_SUBSTEPS], iterations = c.n[N_ITERATIONS];
  const float h = c.f[C_DT] / (float)substeps;
  const float tq = c.f[C_TORQUE];
  const V3 axis = act == 2 ? v3(tq, 0, 0) : act == 3 ? v3(-tq, 0, 0) : act == 4 ? v3(0, 0, tq) : act == 5 ? v3(0, 0, -tq)
                : act == 6 ? v3(0, tq, 0) : act == 7 ? v3(0, -tq, 0) : v3(0, 0, 0);
  const V3 inertia = v3(c.f[C_IX], c.f[C_IY], c.f[C_IZ]);
  for (int s = 0; s < substeps && valid; ++s) {
    float throttle = 0.f;
    V3 torque = v3(0.f, 0.f, 0.f);
    if (act != 0) {
      const float want = (act == 1 ? c.f[C_MAIN_RATE] : c.f[C_ATT_RATE]) * h;
      const float frac = want > 0.f ? fminf(1.f, b.fuel / want) : 1.f;
      const float used = want * frac;
      b.fuel = fmaxf(b.fuel - used, 0.f);
      if (act == 1) { main_used += used; throttle = frac; }
      else { att_used += used; torque = axis * frac; }
    }
    b.throttle = throttle; b.att = torque;
    const V3 thrust = rotate(b.q, v3(0.f, c.f[C_THRUST] * throttle, 0.f));
    b.vel = b.vel + (thrust / c.f[C_MASS] + v3(0.f, -c.f[C_GRAVITY], 0.f)) * h;
    b.pos = b.pos + b.vel * h;
    b.ang = b.ang + (torque - cross(b.ang, inertia * b.ang)) * inverse_inertia(c) * h;
    // q += 0.5 * q * (0, omega) * h, then renormalise
    const Quat q = b.q;
    const V3 w = b.ang;
    Quat dq{-q.x * w.x - q.y * w.y - q.z * w.z, q.w * w.x + q.y * w.z - q.z * w.y, q.w * w.y - q.x * w.z + q.z * w.x,
            q.w * w.z + q.x * w.y - q.y * w.x};
    Quat n{q.w + dq.w * 0.5f * h, q.x + dq.x * 0.5f * h, q.y + dq.y * 0.5f * h, q.z + dq.z * 0.5f * h};
    const float norm = sqrtf(n.w * n.w + n.x * n.x + n.y * n.y + n.z * n.z);
    b.q = Quat{n.w / norm, n.x / norm, n.y / norm, n.z / norm};
    valid = finite_body(b);
    // a lander whose lowest possible point is above the highest terrain vertex touches nothing: skip the contact pass
    const bool airborne = b.pos.y - c.f[C_REACH] > c.f[C_TERRAIN_TOP];
    for (int it = 0; it < iterations && valid && !airborne; ++it) {
      for (int k = 0; k < 7; ++k) resolve_support(c, terrain, b, k, h, d);
      valid = finite_body(b) && isfinite(d.foot_speed);
    }
  }
  if (valid) refresh_contacts(c, terrain, b);
  b.u[U_STEP] += 1;
  bool safe = false;
  if (!valid || !finite_body(b)) { b.u[U_TERM] = 1; b.u[U_REASON] = END_NUMERIC; }
  else if (!ground_at(c, terrain, b.pos.x, b.pos.z).inside || b.pos.y < c.f[C_MIN_Y] || b.pos.y > c.f[C_MAX_Y]) { b.u[U_TERM] = 1; b.u[U_REASON] = END_OOB; }
  else if (d.body_hit || b.u[U_BODY] != 0) { b.u[U_TERM] = 1; b.u[U_REASON] = END_BODY; }
  else if (d.foot_speed > c.f[C_HARD_FOOT]) { b.u[U_TERM] = 1; b.u[U_REASON] = END_HARD_FOOT; }
  else {
    const V3 up = rotate(b.q, v3(0.f, 1.f, 0.f));
    safe = (b.u[U_FOOT] & 15) == 15 && (b.u[U_PAD] & 15) == 15 && b.u[U_BODY] == 0 && length(b.vel) <= c.f[C_SAFE_LIN] &&
           length(b.ang) <= c.f[C_SAFE_ANG] && acosf(fminf(fmaxf(up.y, -1.f), 1.f)) <= c.f[C_SAFE_TILT];
    b.u[U_DWELL] = safe ? b.u[U_DWELL] + 1 : 0;
    if (b.u[U_DWELL] >= c.n[N_DWELL]) { b.u[U_TERM] = 1; b.u[U_REASON] = END_SAFE; }
  }
  if (b.u[U_TERM] == 0 && b.u[U_STEP] >= c.n[N_MAX_STEPS]) { b.u[U_TRUNC] = 1; b.u[U_REASON] = END_TIME; }
  const float pot_after = b.u[U_TERM] != 0 ? 0.f : potential(c, b);
  float soft = 0.f;
  if (d.foot_speed <= c.f[C_HARD_FOOT])
    for (int f = 0; f < 4; ++f)
      if (((b.u[U_FOOT] >> f) & 1) && !((b.u[U_REWARDED] >> f) & 1)) { soft += c.f[C_R_SOFT]; b.u[U_REWARDED] |= 1 << f; }
  const float terminal = b.u[U_REASON] == END_SAFE ? c.f[C_R_SUCCESS] : (b.u[U_TERM] != 0 ? c.f[C_R_FAIL] : 0.f);
  float r = c.f[C_GAMMA] * pot_after - pot_before - c.f[C_W_MAIN_FUEL] * main_used - c.f[C_W_ATT_FUEL] * att_used + soft +
            (safe ? c.f[C_R_DWELL] : 0.f) + terminal;
  float total = b.ret + r;
  if (!isfinite(r) || !isfinite(total)) {
    b.u[U_TERM] = 1; b.u[U_TRUNC] = 0; b.u[U_REASON] = END_NUMERIC;
    r = c.f[C_R_FAIL];
    total = b.ret + r;
    if (!isfinite(total)) total = 0.f;
  }
  b.ret = total;
  store_body(b, sf, su);
  write_observation(c, terrain, b, o);
  reward[e] = r; terminated[e] = b.u[U_TERM] != 0; truncated[e] = b.u[U_TRUNC] != 0; end_reason[e] = b.u[U_REASON];
}

__device__ __forceinline__ unsigned lunar_mix32(unsigned v) {
  v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu; v ^= v >> 16;
  return v;
}
// uniform in [0, 1) from (seed, lane, episode, component): the high 24 bits of the hash
__device__ __forceinline__ float lunar_uniform(unsigned lo, unsigned hi, unsigned env, unsigned episode, unsigned comp) {
  unsigned v = lunar_mix32(lo ^ lunar_mix32(hi + 0x9e3779b9u));
  v = lunar_mix32(v ^ lunar_mix32(env + 0x85ebca6bu));
  v = lunar_mix32(v ^ lunar_mix32(episode + 0xc2b2ae35u));
  v = lunar_mix32(v ^ lunar_mix32(comp + 0x27d4eb2fu));
  return (float)(v >> 8) * (1.0f / 16777216.0f);
}

// spawn = {half extent in x / z, lowest y, highest y, planar speed, descent speed, tilt, yaw, angular speed}
struct Spawn { float v[8]; };

__global__ void __launch_bounds__(128)
lunar_reset_kernel(const Config c, const Spawn sp, const float* __restrict__ terrain, float* __restrict__ state_f, int* __restrict__ state_u,
                   float* __restrict__ obs, int envs, unsigned seed_lo, unsigned seed_hi, int only_done) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= envs) return;
  float* sf = state_f + (long long)e * 32;
  int* su = state_u + (long long)e * 16;
  if (only_done && su[U_TERM] == 0 && su[U_TRUNC] == 0) return;
  const unsigned episode = only_done ? (unsigned)su[U_EPISODE] + 1u : 0u;
  float u[12];
  for (int i = 0; i < 12; ++i) u[i] = lunar_uniform(seed_lo, seed_hi, (unsigned)e, episode, (unsigned)i);
  Body b;
  b.pos = v3((u[0] * 2.f - 1.f) * sp.v[0], sp.v[1] + u[2] * (sp.v[2] - sp.v[1]), (u[1] * 2.f - 1.f) * sp.v[0]);
  b.vel = v3((u[3] * 2.f - 1.f) * sp.v[3], -u[5] * sp.v[4], (u[4] * 2.f - 1.f) * sp.v[3]);
  Quat q{1.f, (u[6] * 2.f - 1.f) * sp.v[5], (u[8] * 2.f - 1.f) * sp.v[6], (u[7] * 2.f - 1.f) * sp.v[5]};
  const float norm = sqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
  b.q = Quat{q.w / norm, q.x / norm, q.y / norm, q.z / norm};
  b.ang = v3((u[9] * 2.f - 1.f) * sp.v[7], (u[10] * 2.f - 1.f) * sp.v[7], (u[11] * 2.f - 1.f) * sp.v[7]);
  b.fuel = c.f[C_FUEL_CAP]; b.throttle = 0.f; b.att = v3(0.f, 0.f, 0.f); b.ret = 0.f;
  for (int i = 0; i < 3; ++i) b.body_imp[i] = 0.f;
  for (int i = 0; i < 4; ++i) b.foot_imp[i] = 0.f;
  for (int i = 0; i < 16; ++i) b.u[i] = 0;
  b.u[U_EPISODE] = (int)episode;
  for (int i = 0; i < 32; ++i) sf[i] = 0.f;
  refresh_contacts(c, terrain, b);
  store_body(b, sf, su);
  write_observation(c, terrain, b, obs + (long long)e * 33);
}

static Config make_config(const float* cfg_f, const int* cfg_n) {
  Config c;
  for (int i = 0; i < C_COUNT; ++i) c.f[i] = cfg_f[i];
  for (int i = 0; i < 6; ++i) c.n[i] = cfg_n[i];
  return c;
}

extern "C" {

// cfg_f: 77 host floats, cfg_n: 6 host ints (see the enums above); everything else is device memory.
int oa_rl_lunar_step(const float* cfg_f, const int* cfg_n, const void* terrain, const void* action, const void* external_stop, void* state_f,
                     void* state_u, void* trans_obs, void* obs, void* reward, void* terminated, void* truncated, void* end_reason, int envs,
                     void* stream) {
  if (envs <= 0 || cfg_n[N_SUBSTEPS] <= 0 || cfg_n[N_CELLS_X] <= 0 || cfg_n[N_CELLS_Z] <= 0) return (int)cudaErrorInvalidValue;
  lunar_step_kernel<<<(envs + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      make_config(cfg_f, cfg_n), (const float*)terrain, (const int*)action, (const unsigned char*)external_stop, (float*)state_f, (int*)state_u,
      (float*)trans_obs, (float*)obs, (float*)reward, (unsigned char*)terminated, (unsigned char*)truncated, (int*)end_reason, envs);
  return (int)cudaGetLastError();
}

int oa_rl_lunar_reset(const float* cfg_f, const int* cfg_n, const float* spawn8, const void* terrain, void* state_f, void* state_u, void* obs,
                      int envs, unsigned seed_lo, unsigned seed_hi, int only_done, void* stream) {
  if (envs <= 0 || cfg_n[N_CELLS_X] <= 0 || cfg_n[N_CELLS_Z] <= 0) return (int)cudaErrorInvalidValue;
  Spawn sp;
  for (int i = 0; i < 8; ++i) sp.v[i] = spawn8[i];
  lunar_reset_kernel<<<(envs + 127) / 128, 128, 0, (cudaStream_t)stream>>>(make_config(cfg_f, cfg_n), sp, (const float*)terrain, (float*)state_f,
                                                                          (int*)state_u, (float*)obs, envs, seed_lo, seed_hi, only_done);
  return (int)cudaGetLastError();
}

}  // extern "C"

}  // namespace oa
