// The VALUE side of the memory chain (head_dim 128, blocks of 128 / 256 tokens), which no later update reads and
// which therefore runs behind the routing kernel, fully parallel:
//
//   kvm_vdelta_kernel   one job per (kv row, update): delta[touched rows x D] = onehot[rows x tokens] x gv[tokens x D]
//                       on the tensor cores, gv = bf16(v * gate) formed in shared memory from the block's values
//                       (tiled TMA), the touched rows compacted onto the 128 accumulator lanes exactly as the routing
//                       kernel compacted them; bf16(delta) goes to the pool row the version table names for
//                       (update, row) -- as an intermediate that the second kernel replaces --, and one bit per
//                       memory row says whether the update touched it.  The jobs are independent: persistent CTAs
//                       take them in turn, the next job's values are in flight while the current one is finished.
//   kvm_vapply_kernel   one warp per memory row walks the updates that touched its row (the bit table), in order:
//                       row = bf16(row + delta), value view = normalize(row) * magnitude written over the delta.
//                       This is the only sequential part (one bf16 rounding per update and row), a few loads and
//                       stores per touched update.
// Follows model/kvm_mixer.py:231-248 (appended rows) and :321-340 (merged values); products of the one-hot
// contraction are exact, its accumulation order is the hardware's and fixed.
#include <algorithm>

#include "kvm_vdelta.cuh"

namespace kvm {
namespace vside {

// The jobs nobody has taken yet (all of them when the routing kernel's launch had no spare CTAs).
__global__ void __launch_bounds__(kThreads, 1)
kvm_vdelta_kernel(const __grid_constant__ DeltaArgs a, const __grid_constant__ Maps maps) {
  extern __shared__ __align__(1024) unsigned char smem[];
  if (*a.status != 0) return;  // the routing kernel gave up: its decisions and version tables are not to be trusted
  delta_jobs(a, maps, smem, threadIdx.x);
}

// ------------------------------------------------------------------------------------------------ apply
constexpr int kApWarps = 8;

// One warp per memory row.  born[row * s_final + r]: the token that created memory row r.
__global__ void __launch_bounds__(kApWarps * 32, 8)
kvm_vapply_kernel(LayerDev L, Tensor4 v, Tensor4 gate, const kvm_update_plan* __restrict__ plan, int n_plan,
                  const int* __restrict__ born, MemoryDev mem, bf16* __restrict__ pool_v, long long pool_rows,
                  const int* __restrict__ ver_idx, long long ver_rows, const unsigned* __restrict__ tbits, int words,
                  int s_final, const int* __restrict__ status) {
  if (*status != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int b = row / L.Hkv, h = row % L.Hkv;
  const int r = blockIdx.x * kApWarps + warp;
  if (r >= s_final) return;
  const int C = L.C, log2c = C == 256 ? 8 : 7;
  const bool versions = pool_v != nullptr && ver_idx != nullptr;
  // ---- the row is born from one token: value (gated where the layer says so) and magnitude
  const int t_b = born[(size_t)row * s_final + r];
  const int u_b = t_b >> log2c;
  float x[4], vl;
  {
    const uint2 raw = *reinterpret_cast<const uint2*>(v.row(b, h, t_b) + lane * 4);
    const float g = __bfloat162float(*gate.row(b, h, t_b));
    const float2 p0 = unpack_bf16(raw.x), p1 = unpack_bf16(raw.y);
    float o[4] = {p0.x, p0.y, p1.x, p1.y};
    const bool gated = u_b == 0 ? (L.gate_initial != 0) : (L.gate_appends != 0 && L.gate_values != 0);
    if (u_b > 0 && gated) {
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = bf16_round(o[e] * g);
    }
    vl = sqrtf(warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]));  // initial rows: of the ungated value
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = (u_b == 0 && gated) ? bf16_round(o[e] * g) : o[e];
  }
  auto view = [&](uint2& o) {  // normalize(row) * magnitude
    const float nrm = fmaxf(sqrtf(warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3])), 1e-12f);
    float y[4] = {x[0], x[1], x[2], x[3]};
    divide_by(y, nrm);
    o.x = pack_bf16(y[0] * vl, y[1] * vl);
    o.y = pack_bf16(y[2] * vl, y[3] * vl);
  };
  const unsigned* bits = tbits + (size_t)row * n_plan * words + (r >> 5);
  const int* ver = ver_idx + (size_t)row * ver_rows + r;
  bf16* pool = pool_v + (size_t)row * pool_rows * HD + lane * 4;
  // ---- the updates from the row's birth on, 32 at a time: which touched the row (one lane per update), then in order
  for (int u0 = u_b; u0 < n_plan; u0 += 32) {
    const int u = u0 + lane;
    bool touched = false;
    int slot = -1;
    if (u < n_plan) {
      touched = u > 0 && ((bits[(size_t)u * words] >> (r & 31)) & 1u);
      if (versions && (touched || u == u_b)) {
        const int vr = plan[u].version_row;
        if (vr >= 0) slot = ver[vr];
      }
    }
    unsigned todo = __ballot_sync(0xffffffffu, touched || u == u_b);
    const unsigned tmask = __ballot_sync(0xffffffffu, touched);
    // the deltas of two touched updates are fetched together (more in flight per warp costs registers, and with them
    // resident warps: a full SM of warps with two loads each hides the latency better than half of one with eight)
    while (todo) {
      constexpr int NB = 2;
      int src[NB], sl[NB];
      uint2 dl[NB];
      int n = 0;
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        src[i] = todo ? __ffs(todo) - 1 : -1;
        if (todo) { todo &= todo - 1; ++n; }
        sl[i] = src[i] >= 0 ? __shfl_sync(0xffffffffu, slot, src[i]) : -1;
        dl[i] = make_uint2(0u, 0u);
        if (src[i] >= 0 && ((tmask >> src[i]) & 1u) && sl[i] >= 0) dl[i] = *reinterpret_cast<const uint2*>(pool + (size_t)sl[i] * HD);
      }
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        if (i < n) {
          if ((tmask >> src[i]) & 1u) {
            const float2 d0 = unpack_bf16(dl[i].x), d1 = unpack_bf16(dl[i].y);
            x[0] = bf16_round(x[0] + d0.x); x[1] = bf16_round(x[1] + d0.y);
            x[2] = bf16_round(x[2] + d1.x); x[3] = bf16_round(x[3] + d1.y);
          }
          if (sl[i] >= 0) {
            uint2 o;
            view(o);
            *reinterpret_cast<uint2*>(pool + (size_t)sl[i] * HD) = o;
          }
        }
      }
    }
  }
  // ---- the carried state and its final view
  const size_t off = ((size_t)row * mem.capacity + r) * HD + lane * 4;
  uint2 s;
  s.x = pack_bf16(x[0], x[1]);
  s.y = pack_bf16(x[2], x[3]);
  *reinterpret_cast<uint2*>(mem.v_sum + off) = s;
  if (lane == 0) mem.vlen[(size_t)row * mem.capacity + r] = vl;
  uint2 o;
  view(o);
  *reinterpret_cast<uint2*>(mem.v_attn + off) = o;
}

}  // namespace vside

// The value side of one batch after the routing kernel: deltas on the tensor cores, then the per-row walk.
// born: [rows][s_max] token that created each memory row; tbits: [rows][n_plan][ceil(s_max / 32)] scratch.
// Tensor map of the values and the arguments of the value-delta jobs (`queue` et al. filled in by the caller).
bool vside_setup(const LayerDev& L, int batch, long long T, Tensor4 v, Tensor4 gate, const kvm_update_plan* plan_dev, int n_plan,
                 int s_max, bf16* pool_v, long long pool_rows, const int* ver_idx, long long ver_rows, const int* route,
                 unsigned* tbits, int* status, uint32_t wait_limit, vside::DeltaArgs* a, vside::Maps* maps) {
  using namespace vside;
  const int C = L.C;
  maps->head_inner = v.sh < v.st ? 1 : 0;
  bool okm;
  if (maps->head_inner) {
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)L.Hkv, (cuuint64_t)T, (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)v.sh * 2, (cuuint64_t)v.st * 2, (cuuint64_t)v.sb * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)C, 1};
    okm = encode_bf16_map(&maps->v, v.ptr, 4, dims, strides, box);
  } else {
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)T, (cuuint64_t)L.Hkv, (cuuint64_t)batch};
    const cuuint64_t strides[3] = {(cuuint64_t)v.st * 2, (cuuint64_t)v.sh * 2, (cuuint64_t)v.sb * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)C, 1, 1};
    okm = encode_bf16_map(&maps->v, v.ptr, 4, dims, strides, box);
  }
  if (!okm) return false;
  a->L = L; a->gate = gate; a->plan = plan_dev; a->n_plan = n_plan; a->rows = batch * L.Hkv; a->route = route;
  a->pool_v = pool_v; a->pool_rows = pool_rows; a->ver_idx = ver_idx; a->ver_rows = ver_rows; a->tbits = tbits;
  a->words = ceil_div(s_max, 32); a->s_max = s_max; a->status = status; a->wait_limit = wait_limit;
  a->queue = nullptr; a->progress = nullptr; a->nc = 1; a->chain_done = nullptr; a->chain_ctas = 0;
  a->given_back = nullptr; a->n_given_back = nullptr; a->given_back_taken = nullptr;
  return true;
}
size_t vside_smem_bytes(int C, int s_max) { return vside::Layout(C, s_max).total; }

// The value side of one batch behind the routing kernel: the value-delta jobs its launch has left (counter `a.queue`),
// then the per-row walk.  born: [rows][s_max] token that created each memory row.
cudaError_t launch_vside(vside::DeltaArgs a, const vside::Maps& maps, Tensor4 v, MemoryDev mem, const int* born, cudaStream_t stream) {
  using namespace vside;
  const int rows = a.rows;
  a.progress = nullptr;  // everything has been published by now
  a.chain_done = nullptr;
  {
    const Layout lay(a.L.C, a.s_max);
    cudaError_t e = cudaFuncSetAttribute(kvm_vdelta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
    if (e != cudaSuccess) return e;
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const int n_jobs = rows * (a.n_plan - 1);
    const int grid = std::max(1, std::min(n_jobs, n_sm));
    kvm_vdelta_kernel<<<grid, kThreads, lay.total, stream>>>(a, maps);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  dim3 agrid((unsigned)ceil_div(a.s_max, kApWarps), rows);
  kvm_vapply_kernel<<<agrid, kApWarps * 32, 0, stream>>>(a.L, v, a.gate, a.plan, a.n_plan, born, mem, a.pool_v, a.pool_rows, a.ver_idx,
                                                         a.ver_rows, a.tbits, a.words, a.s_max, a.status);
  return cudaGetLastError();
}

}  // namespace kvm
