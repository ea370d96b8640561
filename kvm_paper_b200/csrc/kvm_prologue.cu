// Fused prologue of the mixer: everything between the q/k/v/gate projections and the operator's inputs in one pass.
//
// Per token and head: token shift against the previous token, per-head LayerNorm of q and k, rotary embedding,
// the merge gate 1 + elu(.), and (for the keys that a memory update will consume) the prepared key
// bf16(LayerNorm(key with its rotary dims zeroed)) and the gated key bf16(prepared * gate) in the layout the chain
// kernels read, so that the prefill can skip its own pass over the keys.
// Follows model/tokenshift.py:11-37, model/value_residual_mixin.py:219-235 (token shift, ln_q / ln_k),
// model/rwkv7_backbone.py:76-88 (rotary on interleaved pairs), model/kvm_mixer.py:381-399 (merge gate, head-major
// views), model/kvm_mixer.py:120-129 (prepared key).  Every operation of the reference's bf16 module rounds its result
// to bf16; the kernel rounds at the same points.
//
// One group of 8 lanes per (token, head) row, D/8 contiguous elements per lane (16-byte accesses; a rotary pair never
// straddles lanes).  The kernel is a single streaming pass: q, k, v are read once (plus the previous token's
// row, which the neighbouring group has just read: an L1/L2 hit) and written once.
#include "kvm_common.cuh"

namespace kvm {

namespace {

// Lane groups of 8 lanes per row, as in the prefill's own pass over the keys: the prepared keys come out with the same
// bits whichever of the two wrote them.
constexpr int GL = 8;

// Both values rounded to bf16 with one conversion instruction (the kernel is bound by its instruction count).
__device__ __forceinline__ void round2(float& a, float& b) {
  const float2 r = unpack_bf16(pack_bf16(a, b));
  a = r.x;
  b = r.y;
}

// A lane's share of a row as packed bf16 pairs: fetched early, unpacked where it is used (the rotary tables are
// requested together with the row itself, so that their latency is not paid again behind the LayerNorm).
template <int EPL>
__device__ __forceinline__ void load_raw(uint32_t (&w)[EPL / 2], const bf16* p) {
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c) {
      const uint4 u = *reinterpret_cast<const uint4*>(p + c * 8);
      w[c * 4] = u.x; w[c * 4 + 1] = u.y; w[c * 4 + 2] = u.z; w[c * 4 + 3] = u.w;
    }
  } else {
    static_assert(EPL == 4, "lane share of 4 or a multiple of 8 elements");
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    w[0] = u.x; w[1] = u.y;
  }
}

// LayerNorm as the reference's module evaluates it on bf16 rows: moments in fp32, y = (x*rstd - mean*rstd)*w + b with
// every product and sum rounded on its own, one rounding to bf16 at the end.
template <int D>
__device__ __forceinline__ void qk_layer_norm(RowVec<D, GL>& r, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                              int gl) {
  constexpr int EPL = D / GL;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) s += r.x[i];
  const float mean = group_sum<GL>(s) * (1.0f / D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const float d = r.x[i] - mean;
    q += d * d;
  }
  const float var = group_sum<GL>(q) * (1.0f / D);
  const float rstd = 1.0f / sqrtf(fmaxf(var, 0.f) + eps);
  const float bias = __fmul_rn(-mean, rstd);
  // (weights by 16-byte loads: a lane's share starts at a multiple of four elements)
  const float4* w4 = reinterpret_cast<const float4*>(w + gl * EPL);
  const float4* b4 = reinterpret_cast<const float4*>(b + gl * EPL);
#pragma unroll
  for (int i = 0; i < EPL; i += 4) {
    const float4 wv = __ldg(w4 + i / 4), bv = __ldg(b4 + i / 4);
    r.x[i] = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(r.x[i], rstd), bias), wv.x), bv.x);
    r.x[i + 1] = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(r.x[i + 1], rstd), bias), wv.y), bv.y);
    r.x[i + 2] = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(r.x[i + 2], rstd), bias), wv.z), bv.z);
    r.x[i + 3] = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(r.x[i + 3], rstd), bias), wv.w), bv.w);
    round2(r.x[i], r.x[i + 1]);
    round2(r.x[i + 2], r.x[i + 3]);
  }
}

template <int EPL>
__device__ __forceinline__ void store_raw(const uint32_t (&w)[EPL / 2], bf16* p) {
  if constexpr (EPL % 8 == 0) {
#pragma unroll
    for (int c = 0; c < EPL / 8; ++c)
      *reinterpret_cast<uint4*>(p + c * 8) = make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  }
}
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Token shift and rotary embedding are bf16 arithmetic in the reference (every product, difference and sum rounded
// to bf16): they run on packed pairs with the hardware's bf16 instructions (exact result rounded once, which is what
// "compute in fp32, round to bf16" gives for one operation on bf16 operands; the _rn forms are never contracted into
// a fused multiply-add).  Only the LayerNorms unpack to fp32.
template <int D>
__global__ void __launch_bounds__(256)
kvm_prologue_kernel(LayerDev L, PrologueDev p, long long T) {
  constexpr int EPL = D / GL;
  const int gl = threadIdx.x % GL;
  const int HS = L.Hq + 2 * L.Hkv;  // rows per token: query heads, key heads, value heads
  // (the lane groups of a warp reduce with full-warp shuffles: every group runs the same sequence of reductions, on
  // a valid row, and only the stores are predicated)
  const long long unit_raw = (long long)blockIdx.x * (256 / GL) + threadIdx.x / GL;
  const bool valid = unit_raw < T * HS;
  const long long unit = valid ? unit_raw : T * HS - 1;
  const int b = blockIdx.y;
  const long long t = unit / HS;
  const int slot = (int)(unit % HS);
  const int kind = slot < L.Hq ? 0 : (slot < L.Hq + L.Hkv ? 1 : 2);  // q, k, v
  const int h = kind == 0 ? slot : (kind == 1 ? slot - L.Hq : slot - L.Hq - L.Hkv);
  const int H = kind == 0 ? L.Hq : L.Hkv;
  const bf16* lin = kind == 0 ? p.q_lin : (kind == 1 ? p.k_lin : p.v_lin);
  const bf16* shift = kind == 0 ? p.shift_q : (kind == 1 ? p.shift_k : p.shift_v);
  const bf16* prev = kind == 0 ? p.prev_q : (kind == 1 ? p.prev_k : p.prev_v);
  bf16* out = kind == 0 ? p.q_out : (kind == 1 ? p.k_out : p.v_out);
  const size_t row_off = ((size_t)b * T + t) * H * D + (size_t)h * D + gl * EPL;  // this lane's share of the row

  uint32_t x[EPL / 2];
  load_raw<EPL>(x, lin + row_off);
  if (shift) {
    // x + scale * (previous token - x); the first token of a call uses the cached token, or itself
    uint32_t xp[EPL / 2], sc[EPL / 2];
    const bf16* pr = t > 0 ? lin + row_off - (size_t)H * D : (prev ? prev + (size_t)b * H * D + (size_t)h * D + gl * EPL : lin + row_off);
    load_raw<EPL>(xp, pr);
    load_raw<EPL>(sc, shift + (size_t)h * D + gl * EPL);
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      const __nv_bfloat162 xi = as_bf162(x[i]);
      x[i] = as_u32(__hadd2_rn(xi, __hmul2_rn(as_bf162(sc[i]), __hsub2_rn(as_bf162(xp[i]), xi))));
    }
  }
  // (warp-uniform: the reductions inside use full-warp shuffles.  With four or more heads of a kind in a row a warp
  // holds rows of one kind and value rows skip this; in a mixed warp they go through the motions)
  if (p.ln_q_w && __any_sync(0xffffffffu, kind < 2)) {
    RowVec<D, GL> y;
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      const float2 f = unpack_bf16(x[i]);
      y.x[2 * i] = f.x;
      y.x[2 * i + 1] = f.y;
    }
    qk_layer_norm<D>(y, kind == 0 ? p.ln_q_w : p.ln_k_w, kind == 0 ? p.ln_q_b : p.ln_k_b, p.ln_qk_eps, gl);
    if (kind < 2) {
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) x[i] = pack_bf16(y.x[2 * i], y.x[2 * i + 1]);
    }
  }
  if (p.cos != nullptr && kind < 2) {
    uint32_t c[EPL / 2], s[EPL / 2];
    const size_t ro = (size_t)b * p.rope_stride_b + (size_t)t * D + gl * EPL;
    load_raw<EPL>(c, p.cos + ro);
    load_raw<EPL>(s, p.sin + ro);
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {  // cos * x + sin * (pair swapped), the sign of sin folded into the table
      const __nv_bfloat162 xi = as_bf162(x[i]);
      x[i] = as_u32(__hadd2_rn(__hmul2_rn(as_bf162(c[i]), xi), __hmul2_rn(as_bf162(s[i]), __lowhigh2highlow(xi))));
    }
  }
  if (valid) store_raw<EPL>(x, out + row_off);
  const bool is_key = valid && kind == 1;

  // merge gate 1 + elu(g) of this (token, kv head), in the head-major layout [B, Hkv, T]
  float g = 1.0f;
  if (p.gate_lin && is_key) {
    const float gl_in = __bfloat162float(p.gate_lin[((size_t)b * T + t) * L.Hkv + h]);
    const float e = bf16_round(gl_in > 0.f ? gl_in : expf(gl_in) - 1.0f);
    g = bf16_round(1.0f + e);
  }
  if (is_key && gl == 0) p.gate_out[((size_t)b * L.Hkv + h) * T + t] = __float2bfloat16_rn(g);
  const bool consumed = p.pk_all && is_key && t < p.n_tok;
  if (!__any_sync(0xffffffffu, consumed)) return;  // (warp-uniform, as above)
  // prepared key and gated key of a token that a memory update consumes
  RowVec<D, GL> r;
#pragma unroll
  for (int i = 0; i < EPL / 2; ++i) {
    const float2 f = unpack_bf16(x[i]);
    r.x[2 * i] = (gl * EPL + 2 * i < L.rope_dim) ? 0.f : f.x;
    r.x[2 * i + 1] = (gl * EPL + 2 * i + 1 < L.rope_dim) ? 0.f : f.y;
  }
  layer_norm_row_g<D, GL>(r, L.ln_w, L.ln_b, L.ln_eps, gl);
  const size_t po = (((size_t)b * L.Hkv + h) * p.n_tok + t) * D;
  if (consumed) store_row<D, GL>(r, p.pk_all + po, gl);
  if (p.gk_all && consumed) {
    if (L.gate_keys) {
#pragma unroll
      for (int i = 0; i < EPL; i += 2) {
        r.x[i] *= g;
        r.x[i + 1] *= g;
        round2(r.x[i], r.x[i + 1]);
      }
    }
    store_row<D, GL>(r, p.gk_all + po, gl);
  }
}

}  // namespace

cudaError_t launch_prologue(int D, const LayerDev& L, const PrologueDev& p, int batch, long long T, cudaStream_t stream) {
  const long long units = T * (L.Hq + 2 * L.Hkv);
  const dim3 grid((unsigned)((units + 256 / GL - 1) / (256 / GL)), (unsigned)batch);
  switch (D) {
    case 32: kvm_prologue_kernel<32><<<grid, 256, 0, stream>>>(L, p, T); break;
    case 64: kvm_prologue_kernel<64><<<grid, 256, 0, stream>>>(L, p, T); break;
    case 128: kvm_prologue_kernel<128><<<grid, 256, 0, stream>>>(L, p, T); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace kvm
