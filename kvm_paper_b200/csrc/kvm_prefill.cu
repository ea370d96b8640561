#include <algorithm>
// Prefill kernels: (1) the memory chain -- initial memory, then one block-recurrent update per
// token block, each leaving a "version" of the attention view of the memory (an index table into a row pool);
// (2) block attention -- every query tile attends jointly to [memory version ; sliding window]
// with one online softmax (front blocks: plain causal attention over the window only).
//
// The memory trajectory depends only on k, v and the merge gate (model/kvm_mixer.py:478-487), never on
// attention outputs, so the chain runs ahead and attention over all blocks runs in parallel behind it.
#include "kvm_update.cuh"

namespace kvm {

// ------------------------------------------------------------------------------------ prepared keys
// Parallel pre-pass: prepared key (rotary dims zeroed, LayerNorm, bf16) of every token an update will
// consume, written as [kv row][token][D].  Takes the LayerNorm off the sequential chain.
// With `gk_all` it also writes the gated key bf16(pk * gate) of every token (a copy of pk for layers that do not
// gate keys): the tensor-core chain takes both operands of its routing passes from memory.
constexpr int kPrepUnroll = 4;  // tokens per lane group: their loads are issued before the first LayerNorm
template <int D>
__global__ void __launch_bounds__(256)
kvm_prepare_keys_kernel(LayerDev L, Tensor4 k, Tensor4 gate, bf16* __restrict__ pk_all, bf16* __restrict__ gk_all, long long n_tok) {
  constexpr int GL = 8, TPB = 256 / GL;
  const int gl = threadIdx.x % GL;
  const long long base = (long long)blockIdx.x * (TPB * kPrepUnroll) + threadIdx.x / GL;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, h = row % L.Hkv;
  RowVec<D, GL> r[kPrepUnroll];
#pragma unroll
  for (int u = 0; u < kPrepUnroll; ++u) {
    const long long tkn = base + (long long)u * TPB;
    load_row<D, GL>(r[u], k.row(b, h, tkn < n_tok ? tkn : 0), gl);
  }
#pragma unroll
  for (int u = 0; u < kPrepUnroll; ++u) {
    const long long tkn = base + (long long)u * TPB;
#pragma unroll
    for (int i = 0; i < D / GL; ++i)
      if (gl * (D / GL) + i < L.rope_dim) r[u].x[i] = 0.f;
    layer_norm_row<D, GL>(r[u], L.ln_w, L.ln_b, L.ln_eps, gl);
    if (tkn < n_tok) {
      store_row<D, GL>(r[u], pk_all + ((size_t)row * n_tok + tkn) * D, gl);
      if (gk_all) {
        if (L.gate_keys) {
          const float g = __bfloat162float(*gate.row(b, h, tkn));
#pragma unroll
          for (int i = 0; i < D / GL; ++i) r[u].x[i] = bf16_round(r[u].x[i] * g);
        }
        store_row<D, GL>(r[u], gk_all + ((size_t)row * n_tok + tkn) * D, gl);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ chain
// One CTA (or a cluster of up to 4 CTAs) per kv row walks the whole prompt: initial memory, then one update per token block.  The
// attention view of the memory is kept in a row pool with per-version index tables (see ViewStore);
// after the last update the final view is gathered into `mem.k_attn` / `mem.v_attn`.
template <int D, int NT, bool SB>
__global__ void __launch_bounds__(NT, 1)
kvm_chain_kernel(LayerDev L_in, long long T, Tensor4 k, Tensor4 v, Tensor4 gate, const kvm_update_plan* __restrict__ plan,
                 int n_plan, MemoryDev mem, bf16* pool_k, bf16* pool_v, long long pool_rows, int* ver_idx,
                 long long ver_rows, bf16* pk_scr, const bf16* __restrict__ pk_all, int* route, int nc, int* status) {
  extern __shared__ __align__(1024) unsigned char chain_smem[];
  unsigned char* smem_raw = chain_smem;
  // LayerNorm weights in shared memory: almost all of the SM's L1 is carved out as shared memory, so every
  // LayerNorm of the chain would otherwise pay an L2 round trip for them
  __shared__ float ln_s[2 * D];
  for (int i = threadIdx.x; i < D; i += NT) {
    ln_s[i] = L_in.ln_w[i];
    ln_s[D + i] = L_in.ln_b[i];
  }
  LayerDev L = L_in;
  L.ln_w = ln_s;
  L.ln_b = ln_s + D;
  __syncthreads();
  UpdateSmem<D> s;
  s.carve(smem_raw, L.C, mem.capacity, SB);
  s.status = status;
  bool has_tmem = false;
  if constexpr (SB && D == 128 && NT == 512) {
    if (L.C == 128 || L.C == 256) {  // tcgen05 routing scan: its two barriers and tensor memory, once per kernel
      if (threadIdx.x == 0) {
        tc::mbar_init(&s.bars[0], 1);
        tc::mbar_init(&s.bars[1], 1);
        tc::fence_barrier_init();
      }
      if (threadIdx.x < 32) tc::tmem_alloc(reinterpret_cast<uint32_t*>(s.bars + 2), kTcTmemCols);
      has_tmem = true;
      tc::tc_fence_before_sync();
      __syncthreads();
      tc::tc_fence_after_sync();
      s.tmem = *reinterpret_cast<volatile uint32_t*>(s.bars + 2);
      s.use_tc = true;
    }
  }
  const int row = blockIdx.x / nc;     // the nc CTAs of a cluster share one kv row
  const int crank = blockIdx.x % nc;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int tid = threadIdx.x;
  const int C = L.C;
  constexpr int GL = 8;
  constexpr int GROUPS = NT / GL;
  const int gl = tid % GL, grp = tid / GL;

  MemoryRowPtrs m;
  m.k_sum = mem.k_sum + (size_t)row * mem.capacity * D;
  m.v_sum = mem.v_sum + (size_t)row * mem.capacity * D;
  m.vlen = mem.vlen + (size_t)row * mem.capacity;
  m.k_attn = mem.k_attn + (size_t)row * mem.capacity * D;
  m.v_attn = mem.v_attn + (size_t)row * mem.capacity * D;
  bf16* pk = pk_scr + (size_t)row * C * D;
  const bool pool = ver_idx != nullptr;  // some query block reads memory versions
  ViewStore view;
  view.k = pool ? pool_k + (size_t)row * pool_rows * D : m.k_attn;
  view.v = pool ? pool_v + (size_t)row * pool_rows * D : m.v_attn;
  view.cur = pool ? s.cur : nullptr;
  view.pool_next = 0;
  int* my_ver = pool ? ver_idx + (size_t)row * ver_rows : nullptr;

  for (int u = 0; u < n_plan; ++u) {
    const kvm_update_plan pl = plan[u];
    view.ver_idx = (pool && pl.version_row >= 0) ? my_ver + pl.version_row : nullptr;
    if (u == 0) {
      // initial memory: the first min(T,C) tokens row for row (model/kvm_mixer.py:434-447); 8 lanes per row
      const int n0 = pl.n_append;
      for (int base = 0; base < n0; base += GROUPS) {
        const int tkn = base + grp;
        const bool act = tkn < n0;
        const int t_ = act ? tkn : 0;
        RowVec<D, GL> kr, vr;
        prepare_key_row<D, GL>(L, kr, k.row(b, h, t_), gl);
        load_row<D, GL>(vr, v.row(b, h, t_), gl);
        const float vl = row_norm<D, GL>(vr);  // magnitude of the ungated value
        if (L.gate_initial) {
          const float gt = __bfloat162float(*gate.row(b, h, t_));
#pragma unroll
          for (int i = 0; i < D / GL; ++i) {
            kr.x[i] = bf16_round(kr.x[i] * gt);
            vr.x[i] = bf16_round(vr.x[i] * gt);
          }
        }
        const bool mine = act && (t_ % nc == crank);
        if (mine) {
          store_row<D, GL>(kr, m.k_sum + (size_t)t_ * D, gl);
          store_row<D, GL>(vr, m.v_sum + (size_t)t_ * D, gl);
          if (gl == 0) m.vlen[t_] = vl;
        }
        refresh_memory_row<D, GL>(L, kr, vr, vl, view.k + (size_t)t_ * D, view.v + (size_t)t_ * D, gl, mine);
      }
      if (pool)
        for (int i = tid; i < n0; i += NT) s.cur[i] = i;
      view.pool_next = n0;
      if (route && crank == 0)
        for (int i = tid; i < C; i += NT) route[((size_t)row * n_plan) * C + i] = i < n0 ? -(1 + i) : 0;
      if (view.ver_idx && crank == 0)
        for (int i = tid; i < n0; i += NT) view.ver_idx[i] = i;
      __syncthreads();
      if (nc > 1) cluster_sync_all();
    } else {
      TokenSrc src;
      const long long n_tok = (long long)n_plan * C;  // tokens covered by the prepared-key pre-pass
      src.k = pk_all + ((size_t)row * n_tok + (size_t)u * C) * D; src.k_st = D;
      src.v = v.row(b, h, (long long)u * C); src.v_st = v.st;
      src.g = gate.row(b, h, (long long)u * C); src.g_st = gate.st;
      const bool has_next = u + 1 < n_plan;
      src.next_k = has_next ? src.k + (size_t)C * D : nullptr;
      src.next_v = has_next ? v.row(b, h, (long long)(u + 1) * C) : nullptr;
      memory_update<D, NT, SB, true>(L, src, m, view, mem.capacity, pl.state_before, pl.n_append, pk,
                               route ? route + ((size_t)row * n_plan + u) * C : nullptr, s, nc, crank);
    }
  }
  if (pool) {
    // final attention view, row order, for whoever continues from this memory (the decode cache)
    const kvm_update_plan pl = plan[n_plan - 1];
    const int S = pl.state_before + pl.n_append;
    constexpr int CPR = D / 8;
    for (int c = tid + crank * NT; c < S * CPR; c += NT * nc) {
      const int r = c / CPR, cc = c % CPR;
      const size_t src_off = (size_t)s.cur[r] * D + cc * 8;
      *reinterpret_cast<uint4*>(m.k_attn + (size_t)r * D + cc * 8) = *reinterpret_cast<const uint4*>(view.k + src_off);
      *reinterpret_cast<uint4*>(m.v_attn + (size_t)r * D + cc * 8) = *reinterpret_cast<const uint4*>(view.v + src_off);
    }
  }
  if (has_tmem) {
    tc::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) tc::tmem_dealloc(s.tmem, kTcTmemCols);
  }
}

// -------------------------------------------------------------------------------------- attention
constexpr int kAttnBN = 64;  // keys per shared-memory tile

template <int D>
__host__ __device__ constexpr int attn_tile_stride() { return D + 8; }

template <int D>
__host__ __device__ constexpr size_t attn_smem_bytes() {
  return (size_t)2 * 2 * kAttnBN * attn_tile_stride<D>() * sizeof(bf16);
}

// rows [row0, row0+64) of a [*, D] row-major source with row stride `st` elements; rows >= limit zero-filled
template <int D, int NT>
__device__ __forceinline__ void attn_load_tile(bf16* dst, const bf16* src, long long st, long long row0,
                                               long long limit, int tid) {
  constexpr int CPR = D / 8;
  constexpr int STR = attn_tile_stride<D>();
  for (int c = tid; c < kAttnBN * CPR; c += NT) {
    const int r = c / CPR, cc = c % CPR;
    const long long row = row0 + r;
    const bool ok = row < limit;
    cp_async16(dst + r * STR + cc * 8, src + (ok ? row : 0) * st + cc * 8, ok ? 16 : 0);
  }
}

// rows [row0, row0+64) of a memory version: row r lives at pool row idx[r]; rows >= limit zero-filled
template <int D, int NT>
__device__ __forceinline__ void attn_load_tile_idx(bf16* dst, const bf16* pool, const int* __restrict__ idx, int row0,
                                                   int limit, int tid) {
  constexpr int CPR = D / 8;
  constexpr int STR = attn_tile_stride<D>();
  for (int c = tid; c < kAttnBN * CPR; c += NT) {
    const int r = c / CPR, cc = c % CPR;
    const int row = row0 + r;
    const bool ok = row < limit;
    const int slot = ok ? __ldg(idx + row) : 0;
    cp_async16(dst + r * STR + cc * 8, pool + (size_t)slot * D + cc * 8, ok ? 16 : 0);
  }
}

// One CTA = BM query rows of one (batch, q-head) inside one query block j.
template <int D, int BM>
__global__ void __launch_bounds__(BM * 2)
kvm_attn_prefill_kernel(LayerDev L, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                        const kvm_update_plan* __restrict__ plan, const bf16* __restrict__ pool_k,
                        const bf16* __restrict__ pool_v, long long pool_rows, const int* __restrict__ ver_idx,
                        long long ver_rows, bf16* __restrict__ out, int tiles_per_block, int j_begin, float sm_scale,
                        const int* __restrict__ status) {
  if (*status != 0) return;  // an earlier kernel of this prefill gave up: the version tables are not to be trusted
  constexpr int NT = BM * 2;
  constexpr int KS = D / 16;       // k-steps of QK^T
  constexpr int NT8 = kAttnBN / 8; // n8 tiles of a score tile
  constexpr int DT8 = D / 8;       // n8 tiles of the output
  constexpr int STR = attn_tile_stride<D>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);             // [2][64][STR]
  bf16* sV = sK + (size_t)2 * kAttnBN * STR;                // [2][64][STR]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int C = L.C;
  // heavier tiles (later rows of a block see more window keys) are scheduled first
  const int xi = gridDim.x - 1 - blockIdx.x;
  const int j = j_begin + xi / tiles_per_block;
  const int ti = xi % tiles_per_block;
  const int qrow = blockIdx.y;
  const int b = qrow / L.Hq, hq = qrow % L.Hq;
  const int hkv = hq / (L.Hq / L.Hkv);
  const long long q0 = (long long)j * C + (long long)ti * BM;
  const long long q_blk_end = min(T, (long long)(j + 1) * C);
  if (q0 >= q_blk_end) return;
  const long long q_tile_end = min(q_blk_end, q0 + BM);

  // segments
  int S = 0;
  const bf16* mk = nullptr;
  const bf16* mv = nullptr;
  const int* midx = nullptr;
  if (j >= L.W) {
    const kvm_update_plan pl = plan[j - L.W];
    S = pl.state_before + pl.n_append;
    const size_t kvrow = (size_t)(b * L.Hkv + hkv);
    mk = pool_k + kvrow * pool_rows * D;
    mv = pool_v + kvrow * pool_rows * D;
    midx = ver_idx + kvrow * ver_rows + pl.version_row;
  }
  const long long bb = max(0LL, (long long)(j + 1 - L.W) * C);
  const int n_mem_tiles = (S + kAttnBN - 1) / kAttnBN;
  const int n_win_tiles = (int)((q_tile_end - bb + kAttnBN - 1) / kAttnBN);
  const int n_tiles = n_mem_tiles + n_win_tiles;
  const bf16* kbase = k.row(b, hkv, 0);
  const bf16* vbase = v.row(b, hkv, 0);
  const float scale_mem = sm_scale * L.state_temp[hq] * kLog2e;
  const float scale_win = sm_scale * L.front_temp[hq] * kLog2e;

  // Q fragments (rows past the tile end are clamped; their results are never stored)
  uint32_t qa[KS][4];
  const long long qr0 = min(q0 + warp * 16 + g, q_tile_end - 1);
  const long long qr1 = min(q0 + warp * 16 + g + 8, q_tile_end - 1);
  {
    const bf16* p0 = q.row(b, hq, qr0);
    const bf16* p1 = q.row(b, hq, qr1);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c0 = ks * 16 + t * 2;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(p0 + c0);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(p1 + c0);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(p0 + c0 + 8);
      qa[ks][3] = *reinterpret_cast<const uint32_t*>(p1 + c0 + 8);
    }
  }
  const long long qpos0 = q0 + warp * 16 + g, qpos1 = qpos0 + 8;

  float o[DT8][4];
#pragma unroll
  for (int i = 0; i < DT8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  auto issue = [&](int it, int stage) {
    bf16* dK = sK + (size_t)stage * kAttnBN * STR;
    bf16* dV = sV + (size_t)stage * kAttnBN * STR;
    if (it < n_mem_tiles) {
      attn_load_tile_idx<D, NT>(dK, mk, midx, it * kAttnBN, S, tid);
      attn_load_tile_idx<D, NT>(dV, mv, midx, it * kAttnBN, S, tid);
    } else {
      const long long r0 = bb + (long long)(it - n_mem_tiles) * kAttnBN;
      attn_load_tile<D, NT>(dK, kbase, k.st, r0, q_tile_end, tid);
      attn_load_tile<D, NT>(dV, vbase, v.st, r0, q_tile_end, tid);
    }
    cp_async_commit();
  };

  issue(0, 0);
  for (int it = 0; it < n_tiles; ++it) {
    const int cur = it & 1;
    if (it + 1 < n_tiles) {
      issue(it + 1, cur ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* tK = sK + (size_t)cur * kAttnBN * STR;
    const bf16* tV = sV + (size_t)cur * kAttnBN * STR;
    const bool is_mem = it < n_mem_tiles;
    const long long base = is_mem ? (long long)it * kAttnBN : bb + (long long)(it - n_mem_tiles) * kAttnBN;
    const long long limit = is_mem ? (long long)S : q_tile_end;
    const float sc = is_mem ? scale_mem : scale_win;

    // S = Q K^T
    float sacc[NT8][4];
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      const bf16* brow = tK + (size_t)(nt * 8 + g) * STR + t * 2;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + ks * 16);
        uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + ks * 16 + 8);
        mma_bf16_16816(sacc[nt], qa[ks], b0, b1);
      }
    }
    // scale, mask, online softmax (base 2)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const long long n = base + nt * 8 + t * 2 + (e & 1);
        const long long qp = (e >> 1) ? qpos1 : qpos0;
        const bool ok = n < limit && (is_mem || n <= qp);
        const float x = ok ? sacc[nt][e] * sc : -INFINITY;
        sacc[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_use[r]);  // m_run = -inf -> 0
      m_run[r] = m_new;
    }
    uint32_t pa[NT8 / 2][4];
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT8; ++nt) {
      const float p0 = exp2f(sacc[nt][0] - m_use[0]);
      const float p1 = exp2f(sacc[nt][1] - m_use[0]);
      const float p2 = exp2f(sacc[nt][2] - m_use[1]);
      const float p3 = exp2f(sacc[nt][3] - m_use[1]);
      ls[0] += p0 + p1;
      ls[1] += p2 + p3;
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + ls[r];
#pragma unroll
    for (int i = 0; i < DT8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
    // O += P V   (V fragments through transposed ldmatrix: 16 keys x 16 value columns per call)
#pragma unroll
    for (int kk = 0; kk < kAttnBN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DT8 / 2; ++dp) {
        uint32_t vb[4];
        const bf16* vrow = tV + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STR + dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vrow);
        mma_bf16_16816(o[dp * 2 + 0], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[dp * 2 + 1], pa[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();
  }

  // normalise and store [B, T, Hq*D]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
  const float inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
  const long long ostride = (long long)L.Hq * D;
  if (qpos0 < q_tile_end) {
    bf16* p = out + ((long long)b * T + qpos0) * ostride + (long long)hq * D + t * 2;
#pragma unroll
    for (int i = 0; i < DT8; ++i) *reinterpret_cast<uint32_t*>(p + i * 8) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
  }
  if (qpos1 < q_tile_end) {
    bf16* p = out + ((long long)b * T + qpos1) * ostride + (long long)hq * D + t * 2;
#pragma unroll
    for (int i = 0; i < DT8; ++i) *reinterpret_cast<uint32_t*>(p + i * 8) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// ------------------------------------------------------------------------------------- host side
bool chain_tc_supported(int D, const LayerDev& L, int n_plan, int s_max, int rows);
cudaError_t launch_chain_tc(const LayerDev& L, int batch, long long T, Tensor4 v, Tensor4 gate, const kvm_update_plan* plan_dev,
                            int n_plan, int s_max, MemoryDev mem, bf16* pool_k, bf16* pool_v, long long pool_rows, int* ver_idx,
                            long long ver_rows, const bf16* pk_all, const bf16* gk_all, int* route, int* born, unsigned* tbits,
                            int* status, uint32_t wait_limit, uint32_t test_flags, cudaStream_t stream);
cudaError_t launch_attn_tc(const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                           const kvm_update_plan* plan_dev, const bf16* pool_k, const bf16* pool_v, long long pool_rows,
                           const int* ver_idx, long long ver_rows, bf16* out, int* status, cudaStream_t stream,
                           const GatherDst* gd);

template <int D>
static cudaError_t launch_prefill(const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v, Tensor4 gate,
                                  const kvm_update_plan* plan_dev, int n_plan, long long ver_rows, MemoryDev mem,
                                  bf16* out, int* route, bf16* pool_k, bf16* pool_v, long long pool_rows, int* ver_idx,
                                  bf16* pk_scr, bf16* pk_all, bf16* gk_all, int* route_ws, int* born_ws, unsigned* tbits_ws,
                                  int s_final, int* status, unsigned phases, cudaStream_t stream, const GatherDst* gd) {
  constexpr int NT = 512;
  const int rows = batch * L.Hkv;
  const int n_qblocks = (int)((T + L.C - 1) / L.C);
  const bool versions = n_qblocks > L.W && ver_rows > 0;
  cudaError_t e;
  // head_dim 128 and blocks of 128 / 256 tokens: the chain with the resident memory on the tensor cores
  const bool tc_chain = !(phases & KVM_PREFILL_LEGACY_CHAIN) && chain_tc_supported(D, L, n_plan, s_final, rows);
  if ((phases & KVM_PREFILL_CHAIN) && n_plan > 1 && !(phases & KVM_PREFILL_KEYS_PREPARED)) {
    const long long n_tok = (long long)n_plan * L.C;
    dim3 pgrid((unsigned)((n_tok + 32 * kPrepUnroll - 1) / (32 * kPrepUnroll)), rows);
    kvm_prepare_keys_kernel<D><<<pgrid, 256, 0, stream>>>(L, k, gate, pk_all, tc_chain ? gk_all : nullptr, n_tok);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  if ((phases & KVM_PREFILL_CHAIN) && tc_chain) {
    const bool test = (phases & KVM_PREFILL_TEST_WITHHOLD_ARRIVAL) != 0;
    e = launch_chain_tc(L, batch, T, v, gate, plan_dev, n_plan, s_final, mem, pool_k, pool_v, pool_rows, versions ? ver_idx : nullptr,
                        ver_rows, pk_all, gk_all, route ? route : route_ws, born_ws, tbits_ws, status,
                        test ? (1u << 11) : tc::kSpinLimit, test ? 1u : 0u, stream);
    if (e != cudaSuccess) return e;
  } else if (phases & KVM_PREFILL_CHAIN) {
    const bool sb = update_block_fits_smem<D>(L.C, mem.capacity);
    const size_t smem_u = UpdateSmem<D>::bytes(L.C, mem.capacity, sb);
    auto kern = sb ? kvm_chain_kernel<D, NT, true> : kvm_chain_kernel<D, NT, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_u);
    if (e != cudaSuccess) return e;
    // A cluster of CTAs per kv row when the GPU has room for it (the chain is latency-bound per row): the largest
    // cluster size for which every row's cluster is resident at once.  A cluster must fit inside one GPC, so the
    // count of co-resident clusters comes from the occupancy query, not from the SM count alone (16 clusters of 8
    // do not fit 148 SMs: a second wave would double the time).
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem_u;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int nc = 1;
    if (n_plan > 1) {
      // co-resident clusters of 2 and 4 CTAs (the answer depends on the kernel and its shared memory; asked per call:
      // this path serves the less common shapes)
      for (int lg = 2; lg >= 1; --lg) {
        const int c = 1 << lg;
        if (c > kMaxCluster) continue;
        int n_clusters = 0;
        cfg.gridDim = dim3(c * 64);
        attr[0].val.clusterDim.x = c;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, kern, &cfg) != cudaSuccess) {
          (void)cudaGetLastError();
          n_clusters = 0;
        }
        if (n_clusters >= rows) {
          nc = c;
          break;
        }
      }
    }
    cfg.gridDim = dim3(rows * nc);
    attr[0].val.clusterDim.x = nc;
    int* ver_arg = versions ? ver_idx : nullptr;
    e = cudaLaunchKernelEx(&cfg, kern, L, T, k, v, gate, plan_dev, n_plan, mem, pool_k, pool_v, pool_rows, ver_arg, ver_rows,
                           pk_scr, (const bf16*)pk_all, route, nc, status);
    if (e != cudaSuccess) return e;
  }
  if (!(phases & KVM_PREFILL_ATTENTION)) return cudaSuccess;
  if constexpr (D == 128) {
    // tcgen05 / tensor-memory kernel: head_dim 128 and blocks that are whole 128-row query tiles
    if (L.C % 128 == 0 && !(phases & KVM_PREFILL_LEGACY_ATTENTION))
      return launch_attn_tc(L, batch, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx, ver_rows, out, status, stream, gd);
  }

  if (gd) return cudaErrorNotSupported;  // only the tcgen05 attention kernel stores into the other ranks' buffers
  constexpr int BM = 64;
  const int tiles_per_block = (L.C + BM - 1) / BM;
  const size_t smem_a = attn_smem_bytes<D>();
  e = cudaFuncSetAttribute(kvm_attn_prefill_kernel<D, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
  if (e != cudaSuccess) return e;
  dim3 grid(n_qblocks * tiles_per_block, batch * L.Hq);
  kvm_attn_prefill_kernel<D, BM><<<grid, BM * 2, smem_a, stream>>>(L, T, q, k, v, plan_dev, pool_k, pool_v, pool_rows, ver_idx,
                                                                  ver_rows, out, tiles_per_block, 0, 1.0f / sqrtf((float)D), status);
  return cudaGetLastError();
}

cudaError_t prefill_dispatch(int D, const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                             Tensor4 gate, const kvm_update_plan* plan_dev, int n_plan, long long ver_rows,
                             MemoryDev mem, bf16* out, int* route, bf16* pool_k, bf16* pool_v, long long pool_rows,
                             int* ver_idx, bf16* pk_scr, bf16* pk_all, bf16* gk_all, int* route_ws, int* born_ws, unsigned* tbits_ws,
                             int s_final, int* status, unsigned phases, cudaStream_t stream, const GatherDst* gd) {
  switch (D) {
    case 32: return launch_prefill<32>(L, batch, T, q, k, v, gate, plan_dev, n_plan, ver_rows, mem, out, route, pool_k, pool_v, pool_rows, ver_idx, pk_scr, pk_all, gk_all, route_ws, born_ws, tbits_ws, s_final, status, phases, stream, gd);
    case 64: return launch_prefill<64>(L, batch, T, q, k, v, gate, plan_dev, n_plan, ver_rows, mem, out, route, pool_k, pool_v, pool_rows, ver_idx, pk_scr, pk_all, gk_all, route_ws, born_ws, tbits_ws, s_final, status, phases, stream, gd);
    case 128: return launch_prefill<128>(L, batch, T, q, k, v, gate, plan_dev, n_plan, ver_rows, mem, out, route, pool_k, pool_v, pool_rows, ver_idx, pk_scr, pk_all, gk_all, route_ws, born_ws, tbits_ws, s_final, status, phases, stream, gd);
  }
  return cudaErrorInvalidValue;
}


size_t update_smem_bytes(int D, int C, int capacity) {  // of the variant without the staged block
  switch (D) {
    case 32: return UpdateSmem<32>::bytes(C, capacity, false);
    case 64: return UpdateSmem<64>::bytes(C, capacity, false);
    case 128: return UpdateSmem<128>::bytes(C, capacity, false);
  }
  return 0;
}

// ------------------------------------------------------------------------------------ head order after a gather
// src [n_shards][n_tokens][pieces] -> dst [n_tokens][n_shards][pieces], 16-byte pieces: consecutive threads copy
// consecutive pieces of the destination, so both sides move whole runs of `pieces` x 16 bytes.
__global__ void __launch_bounds__(256)
kvm_interleave_shards_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int n_shards, long long n_tokens, int pieces) {
  const long long total = n_tokens * n_shards * pieces;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i % pieces);
    const long long ts = i / pieces;
    const int sh = (int)(ts % n_shards);
    const long long t = ts / n_shards;
    dst[i] = src[((long long)sh * n_tokens + t) * pieces + p];
  }
}

cudaError_t launch_interleave_shards(void* dst, const void* src, int n_shards, long long n_tokens, long long shard_bytes, cudaStream_t stream) {
  const int pieces = (int)(shard_bytes / 16);
  const long long total = n_tokens * n_shards * pieces;
  int dev = 0, n_sm = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)std::min<long long>((total + 255) / 256, (long long)n_sm * 16);
  kvm_interleave_shards_kernel<<<grid, 256, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), n_shards, n_tokens, pieces);
  return cudaGetLastError();
}

}  // namespace kvm
