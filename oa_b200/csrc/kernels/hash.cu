// Batched Keccak: Keccak-f[1600] permutation, SHAKE-128 / SHAKE-256 extendable-output hashing of fixed-length rows, and
// the pairwise SHAKE-256 reduction level of a Merkle tree.  Contract: Source/Public/Oa/Crypto/FnHash.h:21-41 of the
// reference (row i of the output is the hash of row i of the input).  One thread owns one 1600-bit state in registers
// (25 x u64 lanes); the round loop is fully unrolled so rho rotations and pi indices are compile-time constants.
#include "common.cuh"
#include "api.h"

namespace oa {

__constant__ unsigned long long kKeccakRc[24] = {
    0x0000000000000001ull, 0x0000000000008082ull, 0x800000000000808aull, 0x8000000080008000ull, 0x000000000000808bull,
    0x0000000080000001ull, 0x8000000080008081ull, 0x8000000000008009ull, 0x000000000000008aull, 0x0000000000000088ull,
    0x0000000080008009ull, 0x000000008000000aull, 0x000000008000808bull, 0x800000000000008bull, 0x8000000000008089ull,
    0x8000000000008003ull, 0x8000000000008002ull, 0x8000000000000080ull, 0x000000000000800aull, 0x800000008000000aull,
    0x8000000080008081ull, 0x8000000000008080ull, 0x0000000080000001ull, 0x8000000080008008ull};

__device__ __forceinline__ unsigned long long rotl64(unsigned long long v, int n) { return (v << n) | (v >> (64 - n)); }

__device__ __forceinline__ void keccak_f1600(unsigned long long (&a)[25]) {
#pragma unroll 1
  for (int round = 0; round < 24; ++round) {
    unsigned long long c[5], d;
#pragma unroll
    for (int x = 0; x < 5; ++x) c[x] = a[x] ^ a[x + 5] ^ a[x + 10] ^ a[x + 15] ^ a[x + 20];
#pragma unroll
    for (int x = 0; x < 5; ++x) {
      d = c[(x + 4) % 5] ^ rotl64(c[(x + 1) % 5], 1);
#pragma unroll
      for (int y = 0; y < 25; y += 5) a[y + x] ^= d;
    }
    // rho + pi along the 24-lane cycle starting at lane 1
    unsigned long long cur = a[1], t;
#define OA_RP(dst, rot) t = a[dst]; a[dst] = rotl64(cur, rot); cur = t;
    OA_RP(10, 1)  OA_RP(7, 3)   OA_RP(11, 6)  OA_RP(17, 10) OA_RP(18, 15) OA_RP(3, 21)  OA_RP(5, 28)  OA_RP(16, 36)
    OA_RP(8, 45)  OA_RP(21, 55) OA_RP(24, 2)  OA_RP(4, 14)  OA_RP(15, 27) OA_RP(23, 41) OA_RP(19, 56) OA_RP(13, 8)
    OA_RP(12, 25) OA_RP(2, 43)  OA_RP(20, 62) OA_RP(14, 18) OA_RP(22, 39) OA_RP(9, 61)  OA_RP(6, 20)  OA_RP(1, 44)
#undef OA_RP
#pragma unroll
    for (int y = 0; y < 25; y += 5) {
      unsigned long long r0 = a[y], r1 = a[y + 1], r2 = a[y + 2], r3 = a[y + 3], r4 = a[y + 4];
      a[y] = r0 ^ (~r1 & r2); a[y + 1] = r1 ^ (~r2 & r3); a[y + 2] = r2 ^ (~r3 & r4);
      a[y + 3] = r3 ^ (~r4 & r0); a[y + 4] = r4 ^ (~r0 & r1);
    }
    a[0] ^= kKeccakRc[round];
  }
}

__global__ void keccak_f1600_kernel(const unsigned long long* __restrict__ in, unsigned long long* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long a[25];
#pragma unroll
  for (int k = 0; k < 25; ++k) a[k] = in[(long long)i * 25 + k];
  keccak_f1600(a);
#pragma unroll
  for (int k = 0; k < 25; ++k) out[(long long)i * 25 + k] = a[k];
}

// XOR one byte into the little-endian lane array (lane index must be resolved at run time: the state goes through a
// switch-free path by keeping the absorb position in whole lanes where possible)
__device__ __forceinline__ void xor_byte(unsigned long long (&a)[25], int pos, unsigned char v) {
  const unsigned long long w = (unsigned long long)v << (8 * (pos & 7));
  const int lane = pos >> 3;
#pragma unroll
  for (int k = 0; k < 25; ++k) if (k == lane) a[k] ^= w;
}

__device__ __forceinline__ unsigned char get_byte(const unsigned long long (&a)[25], int pos) {
  const int lane = pos >> 3;
  unsigned long long w = 0;
#pragma unroll
  for (int k = 0; k < 25; ++k) if (k == lane) w = a[k];
  return (unsigned char)(w >> (8 * (pos & 7)));
}

// SHAKE with rate `rate` bytes (168 for SHAKE-128, 136 for SHAKE-256): absorb msg_len bytes, pad 0x1F ... 0x80, squeeze
// out_len bytes into a row of out_stride bytes.
__global__ void shake_kernel(const unsigned char* __restrict__ msg, unsigned char* __restrict__ out, int n, int msg_len,
                             int msg_stride, int out_len, int out_stride, int rate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  unsigned long long a[25];
#pragma unroll
  for (int k = 0; k < 25; ++k) a[k] = 0ull;
  const unsigned char* m = msg + (long long)i * msg_stride;
  int pos = 0;
  for (int b = 0; b < msg_len; ++b) {
    xor_byte(a, pos, m[b]);
    if (++pos == rate) { keccak_f1600(a); pos = 0; }
  }
  xor_byte(a, pos, 0x1F);
  xor_byte(a, rate - 1, 0x80);
  keccak_f1600(a);
  unsigned char* o = out + (long long)i * out_stride;
  pos = 0;
  for (int b = 0; b < out_len; ++b) {
    if (pos == rate) { keccak_f1600(a); pos = 0; }
    o[b] = get_byte(a, pos++);
  }
}

// One Merkle level: out[i] = SHAKE256(in[2i] || in[2i+1]) on 32-byte nodes (the last node pairs with itself when the
// level has an odd count).  The 64-byte message fits one rate block, so this is a single permutation per pair.
__global__ void merkle_level_kernel(const unsigned long long* __restrict__ in, unsigned long long* __restrict__ out, int n_in) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_out = (n_in + 1) / 2;
  if (i >= n_out) return;
  const int l = 2 * i, r = min(2 * i + 1, n_in - 1);
  unsigned long long a[25];
#pragma unroll
  for (int k = 0; k < 4; ++k) { a[k] = in[(long long)l * 4 + k]; a[4 + k] = in[(long long)r * 4 + k]; }
#pragma unroll
  for (int k = 8; k < 25; ++k) a[k] = 0ull;
  a[8] ^= 0x1Full;                       // domain separation + first pad bit at byte 64
  a[16] ^= 0x8000000000000000ull;        // last pad bit at byte 135 (rate 136)
  keccak_f1600(a);
#pragma unroll
  for (int k = 0; k < 4; ++k) out[(long long)i * 4 + k] = a[k];
}

}  // namespace oa

using namespace oa;

extern "C" {

int oa_keccak_f1600(const void* in, void* out, int n, void* stream) {
  if (n <= 0) return OA_ERR_ARG;
  keccak_f1600_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const unsigned long long*)in, (unsigned long long*)out, n);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

int oa_shake(int bits, const void* msg, void* out, int n, int msg_len, int msg_stride, int out_len, int out_stride, void* stream) {
  if (n <= 0 || msg_len < 0 || out_len <= 0 || (bits != 128 && bits != 256) || out_stride < out_len) return OA_ERR_ARG;
  shake_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const unsigned char*)msg, (unsigned char*)out, n, msg_len,
                                                                  msg_stride, out_len, out_stride, bits == 128 ? 168 : 136);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

int oa_merkle_level(const void* in, void* out, int n_in, void* stream) {
  if (n_in <= 1) return OA_ERR_ARG;
  const int n_out = (n_in + 1) / 2;
  merkle_level_kernel<<<(n_out + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const unsigned long long*)in, (unsigned long long*)out, n_in);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

}  // extern "C"
