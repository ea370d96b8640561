// Shared device helpers of the KVM kernels (sm_100a): bf16 packing, warp reductions, cp.async,
// warp-level tensor-core MMA wrappers, LayerNorm / value-normalisation of one memory row.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvm_b200.h"

namespace kvm {

typedef __nv_bfloat16 bf16;

constexpr int kWarp = 32;
constexpr float kLog2e = 1.4426950408889634f;

// Device-side copy of kvm_layer (plain values, passed by value to kernels).
struct LayerDev {
  int Hq, Hkv, C, W, rope_dim, sink_len;
  int gate_keys, gate_values, gate_appends, gate_initial;
  float ln_eps;
  const float* ln_w;
  const float* ln_b;
  const float* front_temp;
  const float* state_temp;
};

struct Tensor4 {
  const bf16* ptr;
  long long sb, sh, st;
  __device__ __forceinline__ const bf16* row(int b, int h, long long t) const {
    return ptr + (long long)b * sb + (long long)h * sh + t * st;
  }
};

// Where the block attention of a head-sharded prefill puts its output when it gathers by itself: every rank's
// [B, T, n_ranks * Hq * D] buffer (peer-mapped addresses); this rank's heads go to columns [rank * Hq * D, (rank + 1) * Hq * D)
// of all of them.
struct GatherDst {
  int n_ranks, rank;
  void* base[8];
};

// Arguments of the fused prologue kernel (the projections' outputs, the module's parameters, the outputs).
struct PrologueDev {
  const bf16* q_lin;
  const bf16* k_lin;
  const bf16* v_lin;
  const bf16* gate_lin;
  const bf16* shift_q;
  const bf16* shift_k;
  const bf16* shift_v;
  const bf16* prev_q;
  const bf16* prev_k;
  const bf16* prev_v;
  const float* ln_q_w;
  const float* ln_q_b;
  const float* ln_k_w;
  const float* ln_k_b;
  float ln_qk_eps;
  const bf16* cos;
  const bf16* sin;
  long long rope_stride_b;
  bf16* q_out;
  bf16* k_out;
  bf16* v_out;
  bf16* gate_out;
  bf16* pk_all;
  bf16* gk_all;
  long long n_tok;  // tokens per kv row in pk_all / gk_all
};

struct MemoryDev {
  bf16* k_sum;
  bf16* v_sum;
  float* vlen;
  bf16* k_attn;
  bf16* v_attn;
  int capacity;
};

struct DecodeCacheDev {
  MemoryDev mem;
  bf16* ring_k;
  bf16* ring_v;
  bf16* ring_g;
  int* total_len;
  int* state_len;
};

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// 16-byte async global->shared copy; copies `bytes` (0 or 16) and zero-fills the rest.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four transposed 8x8 bf16 matrices from shared memory (lane l supplies the row address of matrix l/8, row l%8).
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

// Four 8x8 bf16 matrices from shared memory, not transposed (thread (g, t) gets elements [g][2t, 2t+1] of each).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  uint32_t s = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
// Transpose an 8x8 bf16 matrix held one row per lane group (thread (g, t): [g][2t, 2t+1]) across the warp.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------
// One row of D elements is spread over a group of GL lanes (GL = 32: a warp per row; GL = 8: four rows
// per warp): lane l of the group owns the EPL = D/GL contiguous elements [l*EPL, (l+1)*EPL).
template <int GL>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int o = GL / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <int D, int GL = 32>
struct RowVec {
  static constexpr int EPL = D / GL;
  float x[EPL];
};

template <int D, int GL = 32>
__device__ __forceinline__ void load_row(RowVec<D, GL>& r, const bf16* p, int gl) {
  constexpr int EPL = D / GL;
  const bf16* q = p + gl * EPL;
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      uint4 u = *reinterpret_cast<const uint4*>(q + c * 8);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), d = unpack_bf16(u.z), e = unpack_bf16(u.w);
      r.x[c * 8 + 0] = a.x; r.x[c * 8 + 1] = a.y; r.x[c * 8 + 2] = b.x; r.x[c * 8 + 3] = b.y;
      r.x[c * 8 + 4] = d.x; r.x[c * 8 + 5] = d.y; r.x[c * 8 + 6] = e.x; r.x[c * 8 + 7] = e.y;
    }
  } else if constexpr (EPL == 4) {
    uint2 u = *reinterpret_cast<const uint2*>(q);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    r.x[0] = a.x; r.x[1] = a.y; r.x[2] = b.x; r.x[3] = b.y;
  } else if constexpr (EPL == 2) {
    float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(q));
    r.x[0] = a.x; r.x[1] = a.y;
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) r.x[i] = __bfloat162float(q[i]);
  }
}

template <int D, int GL = 32>
__device__ __forceinline__ void store_row(const RowVec<D, GL>& r, bf16* p, int gl) {
  constexpr int EPL = D / GL;
  bf16* q = p + gl * EPL;
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      uint4 u;
      u.x = pack_bf16(r.x[c * 8 + 0], r.x[c * 8 + 1]);
      u.y = pack_bf16(r.x[c * 8 + 2], r.x[c * 8 + 3]);
      u.z = pack_bf16(r.x[c * 8 + 4], r.x[c * 8 + 5]);
      u.w = pack_bf16(r.x[c * 8 + 6], r.x[c * 8 + 7]);
      *reinterpret_cast<uint4*>(q + c * 8) = u;
    }
  } else if constexpr (EPL == 4) {
    uint2 u;
    u.x = pack_bf16(r.x[0], r.x[1]);
    u.y = pack_bf16(r.x[2], r.x[3]);
    *reinterpret_cast<uint2*>(q) = u;
  } else if constexpr (EPL == 2) {
    *reinterpret_cast<uint32_t*>(q) = pack_bf16(r.x[0], r.x[1]);
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) q[i] = __float2bfloat16_rn(r.x[i]);
  }
}

// LayerNorm over the D elements of a row held by a lane group (fp32 statistics, biased variance),
// result rounded to bf16 precision (kept in fp32 registers).
template <int D, int GL = 32>
__device__ __forceinline__ void layer_norm_row(RowVec<D, GL>& r, const float* __restrict__ w,
                                               const float* __restrict__ b, float eps, int gl) {
  constexpr int EPL = D / GL;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) s += r.x[i];
  float mean = group_sum<GL>(s) * (1.0f / D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    float d = r.x[i] - mean;
    q += d * d;
  }
  float var = group_sum<GL>(q) * (1.0f / D);
  float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    int d = gl * EPL + i;
    r.x[i] = bf16_round((r.x[i] - mean) * rstd * w[d] + b[d]);
  }
}

// The same LayerNorm for weights in GLOBAL memory at a 16-byte aligned address (the streaming passes over all keys: the
// prefill's prepared-key pass and the fused prologue, which must give the same bits): weights by 16-byte loads, two
// results rounded per conversion instruction.  The arithmetic per element is that of layer_norm_row.
template <int D, int GL>
__device__ __forceinline__ void layer_norm_row_g(RowVec<D, GL>& r, const float* __restrict__ w, const float* __restrict__ b,
                                                 float eps, int gl) {
  constexpr int EPL = D / GL;
  static_assert(EPL % 4 == 0, "a lane's share starts at a multiple of four elements");
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) s += r.x[i];
  float mean = group_sum<GL>(s) * (1.0f / D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    float d = r.x[i] - mean;
    q += d * d;
  }
  float var = group_sum<GL>(q) * (1.0f / D);
  float rstd = 1.0f / sqrtf(var + eps);
  const float4* w4 = reinterpret_cast<const float4*>(w + gl * EPL);
  const float4* b4 = reinterpret_cast<const float4*>(b + gl * EPL);
#pragma unroll
  for (int i = 0; i < EPL; i += 4) {
    const float4 wv = __ldg(w4 + i / 4), bv = __ldg(b4 + i / 4);
    r.x[i] = (r.x[i] - mean) * rstd * wv.x + bv.x;
    r.x[i + 1] = (r.x[i + 1] - mean) * rstd * wv.y + bv.y;
    r.x[i + 2] = (r.x[i + 2] - mean) * rstd * wv.z + bv.z;
    r.x[i + 3] = (r.x[i + 3] - mean) * rstd * wv.w + bv.w;
    const float2 r01 = unpack_bf16(pack_bf16(r.x[i], r.x[i + 1])), r23 = unpack_bf16(pack_bf16(r.x[i + 2], r.x[i + 3]));
    r.x[i] = r01.x; r.x[i + 1] = r01.y; r.x[i + 2] = r23.x; r.x[i + 3] = r23.y;
  }
}

// L2 norm of a row held by a lane group.
template <int D, int GL = 32>
__device__ __forceinline__ float row_norm(const RowVec<D, GL>& r) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < D / GL; ++i) s += r.x[i] * r.x[i];
  return sqrtf(group_sum<GL>(s));
}

// x[i] / n for one shared divisor: one refined reciprocal, then per element a product and one residual
// correction (the textbook correctly-rounded division with the reciprocal shared across the row).
template <int N>
__device__ __forceinline__ void divide_by(float (&x)[N], float n) {
  const float r0 = __frcp_rn(n);
  const float r = fmaf(fmaf(-n, r0, 1.0f), r0, r0);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    const float q = x[i] * r;
    x[i] = fmaf(fmaf(-q, n, x[i]), r, q);
  }
}

// Attention view of one memory row: k_attn = LN(k_sum), v_attn = v_sum / max(|v_sum|, 1e-12) * vlen.
template <int D, int GL = 32>
__device__ __forceinline__ void refresh_memory_row(const LayerDev& L, RowVec<D, GL> ks, RowVec<D, GL> vs, float vlen,
                                                   bf16* k_attn_row, bf16* v_attn_row, int gl, bool do_store = true) {
  layer_norm_row<D, GL>(ks, L.ln_w, L.ln_b, L.ln_eps, gl);
  float n = fmaxf(row_norm<D, GL>(vs), 1e-12f);
  divide_by(vs.x, n);
#pragma unroll
  for (int i = 0; i < D / GL; ++i) vs.x[i] *= vlen;
  if (do_store) {
    store_row<D, GL>(ks, k_attn_row, gl);
    store_row<D, GL>(vs, v_attn_row, gl);
  }
}

// Prepared key of one token: rotary dims zeroed, LayerNorm, bf16 (model/kvm_mixer.py:120-129).
template <int D, int GL = 32>
__device__ __forceinline__ void prepare_key_row(const LayerDev& L, RowVec<D, GL>& r, const bf16* k_row, int gl) {
  load_row<D, GL>(r, k_row, gl);
#pragma unroll
  for (int i = 0; i < D / GL; ++i)
    if (gl * (D / GL) + i < L.rope_dim) r.x[i] = 0.f;
  layer_norm_row<D, GL>(r, L.ln_w, L.ln_b, L.ln_eps, gl);
}

}  // namespace kvm
