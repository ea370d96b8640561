// Decode kernels: one new token for each of `batch` sequences with ragged lengths.
//   kvm_decode_pre_kernel   per kv row: memory update for sequences whose window start jumps at this
//                           token (one full block leaves the window), direct memory append while the
//                           sequence is shorter than one block, then the ring write of the new token
//   kvm_decode_attn_kernel  persistent joint attention over [memory ; window]: every CTA streams an equal
//                           share of all (sequence, kv head, chunk) triples with 16-byte asynchronous
//                           copies; rows cut by a share boundary are combined by their last CTA, the
//                           last CTA of the launch advances the sequences' lengths
// Follows model/kvm_mixer.py:572-713 (eager single-token step).
#include <algorithm>

#include "kvm_update.cuh"
#include "kvm_tc.cuh"

namespace kvm {

__device__ __forceinline__ int bswa_begin_dev(int total, int C, int W) {
  const int end = ((total + C - 1) / C) * C;
  return max(0, end - W * C);
}

// ------------------------------------------------------------------------------------------- pre
template <int D, int NT, bool UPDATE, bool SB>
__global__ void __launch_bounds__(NT, 1)
kvm_decode_pre_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 k, Tensor4 v, Tensor4 gate,
                      const int* __restrict__ n_append_arr, bf16* pk_scr, int* route) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int row = blockIdx.x;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = L.C, WC = L.W * L.C;
  const int past = cache.total_len[b];
  const int S = cache.state_len[b];
  const int cap = cache.mem.capacity;

  MemoryRowPtrs m;
  m.k_sum = cache.mem.k_sum + (size_t)row * cap * D;
  m.v_sum = cache.mem.v_sum + (size_t)row * cap * D;
  m.vlen = cache.mem.vlen + (size_t)row * cap;
  m.k_attn = cache.mem.k_attn + (size_t)row * cap * D;
  m.v_attn = cache.mem.v_attn + (size_t)row * cap * D;
  bf16* rk = cache.ring_k + (size_t)row * WC * D;
  bf16* rv = cache.ring_v + (size_t)row * WC * D;
  bf16* rg = cache.ring_g + (size_t)row * WC;

  if constexpr (UPDATE) {
    const int n_app = n_append_arr ? n_append_arr[b] : -1;
    if (n_app >= 0) {
      // the block [old_begin, old_begin + C) leaves the window (model/kvm_mixer.py:646-669)
      UpdateSmem<D> s;
      s.carve(smem_raw, C, cap, SB);
      const int old_begin = bswa_begin_dev(past, C, L.W);
      const int slot0 = old_begin % WC;
      TokenSrc src;
      src.k = rk + (size_t)slot0 * D; src.k_st = D;
      src.v = rv + (size_t)slot0 * D; src.v_st = D;
      src.g = rg + slot0; src.g_st = 1;
      src.next_k = nullptr; src.next_v = nullptr;
      ViewStore view;  // decode keeps one live copy of the attention view: rows are refreshed in place
      view.k = m.k_attn; view.v = m.v_attn; view.cur = nullptr; view.ver_idx = nullptr; view.pool_next = 0;
      memory_update<D, NT, SB>(L, src, m, view, cap, S, n_app, pk_scr + (size_t)row * C * D,
                               route ? route + (size_t)row * C : nullptr, s);
    }
  }
  // the new token
  if (warp == 0) {
    const bf16* kp = k.row(b, h, 0);
    const bf16* vp = v.row(b, h, 0);
    const bf16 gt = *gate.row(b, h, 0);
    RowVec<D> kr, vr;
    load_row<D>(kr, kp, lane);
    load_row<D>(vr, vp, lane);
    const int slot = past % WC;
    store_row<D>(kr, rk + (size_t)slot * D, lane);
    store_row<D>(vr, rv + (size_t)slot * D, lane);
    if (lane == 0) rg[slot] = gt;
    if (past < C && S == past && past < cap) {
      // still inside the first block: the token becomes memory row `past` directly
      // (model/kvm_mixer.py:623-638; no gating on this path)
      RowVec<D> pk;
      prepare_key_row<D>(L, pk, kp, lane);
      const float vl = row_norm<D>(vr);
      store_row<D>(pk, m.k_sum + (size_t)past * D, lane);
      store_row<D>(vr, m.v_sum + (size_t)past * D, lane);
      if (lane == 0) m.vlen[past] = vl;
      refresh_memory_row<D>(L, pk, vr, vl, m.k_attn + (size_t)past * D, m.v_attn + (size_t)past * D, lane);
    }
  }
}

// ------------------------------------------------------------------------------------- attention
constexpr int kDecThreads = 128;
constexpr int kDecChunk = 64;        // rows per pipeline stage
constexpr int kDecStages = 3;        // stages per CTA (two in flight while one is consumed)
constexpr int kDecMaxBatch = 1024;   // sequences per launch (their chunk table lives in shared memory)
constexpr int kDecodeRowsPerSplit = 128;  // the workspace holds ceil(max_rows / 128) + 2 partials per query head

template <int D>
__host__ __device__ constexpr int dec_row_stride() { return D + 8; }  // padded rows: conflict-free fragment loads

// Shared-memory layout of the attention kernel (byte offsets), for G query heads per kv head.
struct DecSmem {
  size_t stages, qst, ored, wred, meta, temps, seq, total;
  __host__ __device__ DecSmem(int D, int G, int Hq, int nb) {
    const size_t str = (size_t)(D + 8) * 2;
    size_t off = 0;
    stages = off; off += (size_t)kDecStages * 2 * kDecChunk * str;   // [stage][K | V][row][padded D] bf16
    qst = off;    off += (size_t)kDecStages * G * str;               // [stage][query head][padded D] bf16
    ored = off;   off += (size_t)4 * G * D * 4;                      // [warp][query head][D] fp32
    wred = off;   off += (size_t)2 * 4 * 16 * 4;                     // per-warp running max / sum
    meta = off;   off += (size_t)kDecStages * 32;                    // per-stage chunk description (8 ints)
    temps = off;  off += (size_t)2 * Hq * 4;                         // folded softmax scales per query head
    seq = off;    off += (size_t)(3 * nb + 4) * 4;                   // per sequence: S, total, chunk prefix
    total = (off + 15) & ~(size_t)15;
  }
};

// Chunk geometry of one sequence's kv rows: up to three contiguous runs (memory rows, window part up to
// the end of the ring, wrapped window part), each cut into chunks of kDecChunk rows.
struct DecGeo {
  int S_act, slot0, len_a, len_b, c_mem, c_a, c_b;
  __device__ __forceinline__ int chunks() const { return c_mem + c_a + c_b; }
};
__device__ __forceinline__ DecGeo dec_geometry(int S, int total, int C, int W) {
  DecGeo g;
  const int WC = W * C;
  const int new_begin = bswa_begin_dev(total, C, W);
  g.S_act = new_begin > 0 ? S : 0;
  const int n_win = total - new_begin;
  g.slot0 = new_begin % WC;
  g.len_a = min(n_win, WC - g.slot0);
  g.len_b = n_win - g.len_a;
  g.c_mem = (g.S_act + kDecChunk - 1) / kDecChunk;
  g.c_a = (g.len_a + kDecChunk - 1) / kDecChunk;
  g.c_b = (g.len_b + kDecChunk - 1) / kDecChunk;
  return g;
}

// Joint attention of one new token per sequence over [memory ; window], persistent and bandwidth-bound.
// All (sequence, kv head, chunk) triples of the launch form one flat list (sequence-major); every CTA
// takes an equal contiguous range of it and streams the range through a ring of kDecStages shared-memory
// stages with coalesced 16-byte asynchronous copies (a warp moves 512 contiguous bytes per instruction)
// into padded rows.  The copies run two chunks ahead of the math and do not stop at row boundaries, so
// 64 KB per CTA (two CTAs per SM) are in flight from the first to the last chunk of the CTA.
// All query heads of a kv head (G <= 16) form the M=16 tile of warp-level MMAs; each warp owns 16 keys of
// every chunk and keeps a running (max, sum, output) that is merged across the warps when the CTA leaves
// the kv row.  A row that lies inside one CTA's range is finished there; a row cut by a range boundary
// leaves partial results [m, l, acc[D]] (fp32) and the last of its CTAs combines them.  The last CTA of
// the launch advances the lengths of the sequences it covered (nobody reads them any more by then).
// `mode`: 0 = all sequences, 1 = only sequences without a memory update at this token, 2 = only those with.
template <int D>
__global__ void __launch_bounds__(kDecThreads, 2)
kvm_decode_attn_kernel(LayerDev L, DecodeCacheDev cache, Tensor4 q, const int* __restrict__ n_append_arr,
                       float* __restrict__ partial, int* __restrict__ row_counters, int* __restrict__ done_counter,
                       bf16* __restrict__ out, float sm_scale, int b0, int nb, int nslots, int per_min, int mode) {
  constexpr int STR = dec_row_stride<D>();
  constexpr int KS = D / 16;   // k-steps of Q K^T
  constexpr int DT8 = D / 8;   // n8 tiles of the output
  constexpr int CH = kDecChunk, ST = kDecStages;
  constexpr int CPR = D / 8;                      // 16-byte pieces per row
  constexpr int RPI = kDecThreads / CPR;          // rows per pass of the CTA
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int G = L.Hq / L.Hkv, Hkv = L.Hkv;
  const DecSmem lay(D, G, L.Hq, nb);
  bf16* stage0 = reinterpret_cast<bf16*>(smem_raw + lay.stages);
  bf16* qst = reinterpret_cast<bf16*>(smem_raw + lay.qst);
  float* ored = reinterpret_cast<float*>(smem_raw + lay.ored);
  float* wmax = reinterpret_cast<float*>(smem_raw + lay.wred);
  float* wsum = wmax + 64;
  int* meta = reinterpret_cast<int*>(smem_raw + lay.meta);          // [ST][8]
  float* temp_mem = reinterpret_cast<float*>(smem_raw + lay.temps);  // [Hq]
  float* temp_win = temp_mem + L.Hq;                                 // [Hq]
  int* sq_S = reinterpret_cast<int*>(smem_raw + lay.seq);            // [nb]
  int* sq_tot = sq_S + nb;                                           // [nb]
  int* cpre = sq_tot + nb;                                           // [nb + 1] chunks per kv row, prefix
  __shared__ int s_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int C = L.C, W = L.W, WC = L.W * L.C;
  const int cap = cache.mem.capacity;

  // ---- setup: lengths of the sequences in scope, their chunk counts, the prefix over sequences
  for (int b = tid; b < nb; b += kDecThreads) {
    const int B = b0 + b;
    const int n_app = n_append_arr ? n_append_arr[B] : -1;
    const bool in_scope = mode == 0 || (mode == 1 && n_app < 0) || (mode == 2 && n_app >= 0);
    int cnt = 0, S = 0, total = 0;
    if (in_scope) {
      const int past = cache.total_len[B];
      S = cache.state_len[B] + (n_app > 0 ? n_app : 0);
      if (past < C && S == past) S += 1;  // direct append done by the pre kernel
      total = past + 1;
      cnt = dec_geometry(S, total, C, W).chunks();
    }
    sq_S[b] = S;
    sq_tot[b] = total;
    cpre[b + 1] = cnt;
  }
  for (int h = tid; h < L.Hq; h += kDecThreads) {
    temp_mem[h] = sm_scale * L.state_temp[h] * kLog2e;
    temp_win[h] = sm_scale * L.front_temp[h] * kLog2e;
  }
  if (tid == 0) cpre[0] = 0;
  __syncthreads();
  if (warp == 0) {  // inclusive scan of cpre[1..nb], 32 entries at a time
    int carry = 0;
    for (int base = 0; base < nb; base += 32) {
      const int i = base + lane;
      int x = i < nb ? cpre[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      if (i < nb) cpre[i + 1] = x + carry;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
  }
  __syncthreads();
  const int total_f = cpre[nb] * Hkv;                         // chunks of the launch
  const int per = max(per_min, (total_f + (int)gridDim.x - 1) / (int)gridDim.x);
  const int active = (total_f + per - 1) / per;               // CTAs with work
  const int cta = blockIdx.x;
  if (cta >= active) return;
  const int f_begin = cta * per, f_end = min(total_f, f_begin + per);
  const int nloc = f_end - f_begin;

  // ---- producer cursor: (sequence, kv head, chunk) of the next chunk to fetch
  int pb, ph, pc, pcb;
  DecGeo pg;
  {
    int lo = 0, hi = nb - 1;  // last b with cpre[b] * Hkv <= f_begin and a non-empty range
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (cpre[mid] * Hkv <= f_begin) lo = mid; else hi = mid - 1;
    }
    pb = lo;
    pcb = cpre[pb + 1] - cpre[pb];
    const int rem = f_begin - cpre[pb] * Hkv;
    ph = rem / pcb;
    pc = rem - ph * pcb;
    pg = dec_geometry(sq_S[pb], sq_tot[pb], C, W);
  }
  const int my_c = tid % CPR, my_r = tid / CPR;
  // Fetch the producer cursor's chunk into stage s (local chunk index i) and advance the cursor.
  auto issue = [&](int i, int s) {
    const int row = (b0 + pb) * Hkv + ph;
    int n;
    size_t r0;
    const bf16 *bk, *bv;
    const bool is_mem = pc < pg.c_mem;
    if (is_mem) {
      n = min(CH, pg.S_act - pc * CH);
      r0 = (size_t)row * cap + (size_t)pc * CH;
      bk = cache.mem.k_attn;
      bv = cache.mem.v_attn;
    } else if (pc < pg.c_mem + pg.c_a) {
      const int c = pc - pg.c_mem;
      n = min(CH, pg.len_a - c * CH);
      r0 = (size_t)row * WC + pg.slot0 + (size_t)c * CH;
      bk = cache.ring_k;
      bv = cache.ring_v;
    } else {
      const int c = pc - pg.c_mem - pg.c_a;
      n = min(CH, pg.len_b - c * CH);
      r0 = (size_t)row * WC + (size_t)c * CH;
      bk = cache.ring_k;
      bv = cache.ring_v;
    }
    const bool first = i == 0 || pc == 0;
    const bool last = i == nloc - 1 || pc == pcb - 1;
    bf16* dk = stage0 + (size_t)(s * 2) * CH * STR + my_c * 8;
    bf16* dv = dk + (size_t)CH * STR;
    const bf16* gk = bk + r0 * D + my_c * 8;
    const bf16* gv = bv + r0 * D + my_c * 8;
#pragma unroll
    for (int k2 = 0; k2 < CH / RPI; ++k2) {
      const int r = my_r + k2 * RPI;
      const bool in = r < n;  // rows past the run: zero-filled (scores masked, values must be finite)
      const size_t go = (size_t)(in ? r : 0) * D;
      cp_async16(dk + (size_t)r * STR, gk + go, in ? 16 : 0);
      cp_async16(dv + (size_t)r * STR, gv + go, in ? 16 : 0);
    }
    if (first) {  // the query rows of this kv head travel with the first chunk of the row segment
      for (int p = tid; p < G * CPR; p += kDecThreads) {
        const int qh = p / CPR, c8 = p - qh * CPR;
        cp_async16(qst + ((size_t)s * G + qh) * STR + c8 * 8, q.row(b0 + pb, ph * G + qh, 0) + c8 * 8, 16);
      }
    }
    if (tid == 0) {
      int seg = 0, nsegs = 1;
      if (last) {
        const int row_f = cpre[pb] * Hkv + ph * pcb;  // flat index of the row's first chunk
        const int first_cta = row_f / per;
        seg = cta - first_cta;
        nsegs = (row_f + pcb - 1) / per - first_cta + 1;
      }
      int* m = meta + s * 8;
      m[0] = n | (is_mem ? 1 << 16 : 0) | (first ? 1 << 17 : 0) | (last ? 1 << 18 : 0);
      m[1] = row;
      m[2] = seg;
      m[3] = nsegs;
    }
    // advance
    if (++pc == pcb) {
      pc = 0;
      if (++ph == Hkv) {
        ph = 0;
        ++pb;
        while (pb < nb && cpre[pb + 1] == cpre[pb]) ++pb;
        if (pb < nb) {
          pcb = cpre[pb + 1] - cpre[pb];
          pg = dec_geometry(sq_S[pb], sq_tot[pb], C, W);
        }
      }
    }
  };

  // prologue: the first ST-1 chunks in flight (one commit group per chunk, empty groups keep the count uniform)
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < nloc) issue(s, s);
    cp_async_commit();
  }

  uint32_t qa[KS][4];
  float scl_mem[2] = {0.f, 0.f}, scl_win[2] = {0.f, 0.f};
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[DT8][4];

  for (int i = 0; i < nloc; ++i) {
    const int s = i % ST;
    cp_async_wait<ST - 2>();  // this thread's pieces of chunk i have landed
    __syncthreads();          // ... everybody's have, and everybody is done with the stage refilled next
    if (i + ST - 1 < nloc) issue(i + ST - 1, (i + ST - 1) % ST);
    cp_async_commit();

    const int4 md = *reinterpret_cast<const int4*>(meta + s * 8);
    const int n = md.x & 0xffff;
    const bool is_mem = (md.x >> 16) & 1, first = (md.x >> 17) & 1, last = (md.x >> 18) & 1;
    const int row = md.y;
    const int hkv = row % Hkv;
    if (first) {  // new kv row (or the CTA's first chunk): reset the running state, fetch the query fragments
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        m_row[r] = -INFINITY;
        l_row[r] = 0.f;
        const int qh = g + r * 8;
        const bool okq = qh < G;
        const int hq = hkv * G + (okq ? qh : 0);
        scl_mem[r] = temp_mem[hq];
        scl_win[r] = temp_win[hq];
        const bf16* qp = qst + ((size_t)s * G + (okq ? qh : 0)) * STR + t * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          qa[ks][r] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
          qa[ks][2 + r] = okq ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
        }
      }
#pragma unroll
      for (int d8 = 0; d8 < DT8; ++d8) o[d8][0] = o[d8][1] = o[d8][2] = o[d8][3] = 0.f;
    }
    {
      const bf16* sK = stage0 + (size_t)(s * 2) * CH * STR;
      const bf16* sV = sK + (size_t)CH * STR;
      // S = Q K^T for this warp's 16 keys of the chunk
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
        const bf16* brow = sK + (size_t)(warp * 16 + j * 8 + g) * STR + t * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const uint32_t b0r = *reinterpret_cast<const uint32_t*>(brow + ks * 16);
          const uint32_t b1r = *reinterpret_cast<const uint32_t*>(brow + ks * 16 + 8);
          mma_bf16_16816(sacc[j], qa[ks], b0r, b1r);
        }
      }
      const float sc0 = is_mem ? scl_mem[0] : scl_win[0], sc1 = is_mem ? scl_mem[1] : scl_win[1];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = warp * 16 + j * 8 + t * 2 + (e & 1);
          const float x = key < n ? sacc[j][e] * ((e >> 1) ? sc1 : sc0) : -INFINITY;
          sacc[j][e] = x;
          mx[e >> 1] = fmaxf(mx[e >> 1], x);
        }
      }
      bool grew = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        grew = grew || mx[r] > m_row[r];
      }
      if (__any_sync(0xffffffffu, grew)) {  // running maximum moved: rescale what has been accumulated
        float f[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float mn = fmaxf(m_row[r], mx[r]);
          f[r] = m_row[r] == -INFINITY ? 0.f : exp2f(m_row[r] - mn);
          m_row[r] = mn;
          l_row[r] *= f[r];
        }
#pragma unroll
        for (int d8 = 0; d8 < DT8; ++d8) {
          o[d8][0] *= f[0];
          o[d8][1] *= f[0];
          o[d8][2] *= f[1];
          o[d8][3] *= f[1];
        }
      }
      const float mu0 = m_row[0] == -INFINITY ? 0.f : m_row[0];
      const float mu1 = m_row[1] == -INFINITY ? 0.f : m_row[1];
      // P = exp2(S - m) and O += P V for this warp's keys
      uint32_t pa[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = exp2f(sacc[j][0] - mu0), p1 = exp2f(sacc[j][1] - mu0);
        const float p2 = exp2f(sacc[j][2] - mu1), p3 = exp2f(sacc[j][3] - mu1);
        l_row[0] += p0 + p1;
        l_row[1] += p2 + p3;
        pa[j * 2 + 0] = pack_bf16(p0, p1);
        pa[j * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int dp = 0; dp < DT8 / 2; ++dp) {
        uint32_t vb[4];
        const bf16* vrow = sV + (size_t)(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STR + dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vrow);
        mma_bf16_16816(o[dp * 2 + 0], pa, vb[0], vb[1]);
        mma_bf16_16816(o[dp * 2 + 1], pa, vb[2], vb[3]);
      }
    }
    if (!last) continue;

    // ---- the CTA leaves this kv row: merge the four warps' running states
    const int seg = md.z, nsegs = md.w;
    const int b = row / Hkv;  // absolute sequence index
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_row[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t == 0) {
        wmax[warp * 16 + g + r * 8] = m_row[r];
        wsum[warp * 16 + g + r * 8] = l;
      }
      const int qh = g + r * 8;
      if (qh < G) {
        float* dst = ored + ((size_t)warp * G + qh) * D + t * 2;
#pragma unroll
        for (int d8 = 0; d8 < DT8; ++d8) *reinterpret_cast<float2*>(dst + d8 * 8) = make_float2(o[d8][r * 2], o[d8][r * 2 + 1]);
      }
    }
    __syncthreads();
    for (int gq = 0; gq < G; ++gq) {
      const int hq = hkv * G + gq;
      const float M = fmaxf(fmaxf(wmax[gq], wmax[16 + gq]), fmaxf(wmax[32 + gq], wmax[48 + gq]));
      float f[4], lsum = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        f[w] = wmax[w * 16 + gq] == -INFINITY ? 0.f : exp2f(wmax[w * 16 + gq] - M);
        lsum += f[w] * wsum[w * 16 + gq];
      }
      float acc = 0.f;
      if (tid < D) {
        const float* src = ored + (size_t)gq * D + tid;
        acc = f[0] * src[0] + f[1] * src[(size_t)G * D] + f[2] * src[(size_t)2 * G * D] + f[3] * src[(size_t)3 * G * D];
      }
      if (nsegs == 1) {  // the whole row was here
        if (tid < D) out[(size_t)b * L.Hq * D + (size_t)hq * D + tid] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
      } else {
        float* pout = partial + ((size_t)(b * L.Hq + hq) * nslots + seg) * (D + 2);
        if (tid < D) pout[2 + tid] = acc;
        if (tid == 0) {
          pout[0] = M;
          pout[1] = lsum;
        }
      }
    }
    if (nsegs > 1) {  // the last CTA of this kv row combines the partial results
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int prev = atomicAdd(&row_counters[row], 1);
        s_flag = (prev == nsegs - 1);
      }
      __syncthreads();
      if (s_flag) {
        __threadfence();
        for (int gq = 0; gq < G; ++gq) {
          const int hq = hkv * G + gq;
          const float* pin = partial + ((size_t)(b * L.Hq + hq) * nslots) * (D + 2);
          float M = -INFINITY;
          for (int s2 = 0; s2 < nsegs; ++s2) M = fmaxf(M, __ldcg(pin + (size_t)s2 * (D + 2)));
          if (tid < D) {
            float Lsum = 0.f, a = 0.f;
            for (int s2 = 0; s2 < nsegs; ++s2) {
              const float ms = __ldcg(pin + (size_t)s2 * (D + 2));
              const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
              Lsum += w * __ldcg(pin + (size_t)s2 * (D + 2) + 1);
              a += w * __ldcg(pin + (size_t)s2 * (D + 2) + 2 + tid);
            }
            out[(size_t)b * L.Hq * D + (size_t)hq * D + tid] = __float2bfloat16_rn(Lsum > 0.f ? a / Lsum : 0.f);
          }
        }
        if (tid == 0) row_counters[row] = 0;
      }
    }
  }
  cp_async_wait<0>();

  // ---- the last CTA of the launch advances the lengths of the sequences in scope
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int prev = atomicAdd(done_counter, 1);
    s_flag = (prev == active - 1);
  }
  __syncthreads();
  if (s_flag) {
    for (int b = tid; b < nb; b += kDecThreads) {
      if (cpre[b + 1] != cpre[b]) {
        cache.total_len[b0 + b] = sq_tot[b];
        cache.state_len[b0 + b] = sq_S[b];
      }
    }
    if (tid == 0) *done_counter = 0;
  }
}

// Rebuild the attention view of rows [0, state_len[b]) from the carried sums.
template <int D>
__global__ void kvm_memory_refresh_kernel(LayerDev L, MemoryDev mem, const int* __restrict__ state_len) {
  const int row = blockIdx.y;
  const int b = row / L.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;
  if (r >= state_len[b] || r >= mem.capacity) return;
  const size_t off = ((size_t)row * mem.capacity + r) * D;
  RowVec<D> ks, vs;
  load_row<D>(ks, mem.k_sum + off, lane);
  load_row<D>(vs, mem.v_sum + off, lane);
  refresh_memory_row<D>(L, ks, vs, mem.vlen[(size_t)row * mem.capacity + r], mem.k_attn + off, mem.v_attn + off, lane);
}

// ------------------------------------------------------------------------------------- host side
static int device_sm_count() {
  int dev = 0, n_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n_sm <= 0)
    return 148;
  return n_sm;
}

template <int D>
static cudaError_t launch_decode(const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                                 Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                                 int* route, bf16* pk_scr, bf16* gk_scr, float* partial, int* counters,
                                 int rows_per_split, cudaStream_t stream) {
  constexpr int NT = 512;
  const int rows = batch * L.Hkv;
  cudaError_t e;
  if (any_update) {
    const bool sb = update_block_fits_smem<D>(L.C, cache.mem.capacity);
    const size_t smem_u = UpdateSmem<D>::bytes(L.C, cache.mem.capacity, sb);
    auto kern = sb ? kvm_decode_pre_kernel<D, NT, true, true> : kvm_decode_pre_kernel<D, NT, true, false>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_u);
    if (e != cudaSuccess) return e;
    kern<<<rows, NT, smem_u, stream>>>(L, cache, k, v, gate, n_append, pk_scr, route);
  } else {
    kvm_decode_pre_kernel<D, 32, false, false><<<rows, 32, 0, stream>>>(L, cache, k, v, gate, nullptr, pk_scr, route);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // The workspace holds `nslots` partial results per query head; a kv row of at most max_chunks chunks cut
  // into ranges of at least per_min chunks never needs more.
  (void)rows_per_split;
  (void)gk_scr;
  const int G = L.Hq / L.Hkv;
  if (G > 16) return cudaErrorInvalidValue;  // the query heads of a kv head form one M=16 MMA tile
  const int nslots = (max_rows + kDecodeRowsPerSplit - 1) / kDecodeRowsPerSplit + 2;
  const int max_chunks = (max_rows + kDecChunk - 1) / kDecChunk + 3;
  const int per_min = (max_chunks + nslots - 2) / (nslots - 1);
  auto kern = kvm_decode_attn_kernel<D>;
  static size_t smem_set = 0, occ_smem = 0;  // largest dynamic shared memory enabled so far; occupancy cache
  static int occ_cached = 0, dev_set = -1;
  int dev_now = 0;
  cudaGetDevice(&dev_now);
  if (dev_now != dev_set) {  // function attributes are per device
    smem_set = occ_smem = 0;
    dev_set = dev_now;
  }
  for (int b0 = 0; b0 < batch; b0 += kDecMaxBatch) {
    const int nb = std::min(kDecMaxBatch, batch - b0);
    const DecSmem lay(D, G, L.Hq, nb);
    if (lay.total > smem_set) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
      if (e != cudaSuccess) return e;
      smem_set = lay.total;
    }
    if (occ_smem != lay.total) {
      int occ = 0;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kDecThreads, lay.total);
      if (e != cudaSuccess) return e;
      occ_cached = std::max(1, occ);
      occ_smem = lay.total;
    }
    const int grid = occ_cached * device_sm_count();
    kern<<<grid, kDecThreads, lay.total, stream>>>(L, cache, q, any_update ? n_append : nullptr, partial, counters,
                                                   counters + rows, out, 1.0f / sqrtf((float)D), b0, nb, nslots, per_min, 0);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t decode_dispatch(int D, const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                            Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                            int* route, bf16* pk_scr, bf16* gk_scr, float* partial, int* counters, int rows_per_split,
                            cudaStream_t stream) {
  switch (D) {
    case 32: return launch_decode<32>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
    case 64: return launch_decode<64>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
    case 128: return launch_decode<128>(L, batch, cache, q, k, v, gate, n_append, any_update, max_rows, out, route, pk_scr, gk_scr, partial, counters, rows_per_split, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t refresh_dispatch(int D, const LayerDev& L, int batch, MemoryDev mem, const int* state_len, cudaStream_t stream) {
  dim3 grid((mem.capacity + 7) / 8, batch * L.Hkv);
  switch (D) {
    case 32: kvm_memory_refresh_kernel<32><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 64: kvm_memory_refresh_kernel<64><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    case 128: kvm_memory_refresh_kernel<128><<<grid, 256, 0, stream>>>(L, mem, state_len); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace kvm
