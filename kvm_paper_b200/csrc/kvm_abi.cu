// extern "C" entry points of libkvm_b200: argument validation, workspace carve-up, launches.
// Nothing here allocates device memory.  What the library keeps between calls is listed in the header.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "kvm_common.cuh"

namespace kvm {
cudaError_t prefill_dispatch(int D, const LayerDev& L, int batch, long long T, Tensor4 q, Tensor4 k, Tensor4 v,
                             Tensor4 gate, const kvm_update_plan* plan_dev, int n_plan, long long ver_rows,
                             MemoryDev mem, bf16* out, int* route, bf16* pool_k, bf16* pool_v, long long pool_rows,
                             int* ver_idx, bf16* pk_scr, bf16* pk_all, bf16* gk_all, int* route_ws, int* born_ws, unsigned* tbits_ws,
                             int s_final, int* status, unsigned phases, cudaStream_t stream, const kvm::GatherDst* gd);
size_t update_smem_bytes(int D, int C, int capacity);
cudaError_t decode_dispatch(int D, const LayerDev& L, int batch, const DecodeCacheDev& cache, Tensor4 q, Tensor4 k,
                            Tensor4 v, Tensor4 gate, const int* n_append, int any_update, int max_rows, bf16* out,
                            int* route, bf16* pk_scr, float* partial, int* counters, int nslots, int overlap,
                            cudaStream_t stream);
cudaError_t refresh_dispatch(int D, const LayerDev& L, int batch, MemoryDev mem, const int* state_len,
                             cudaStream_t stream);
}  // namespace kvm

using namespace kvm;

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* where) {
  return fail(KVM_ERR_CUDA, "%s: CUDA error %d (%s)", where, (int)e, cudaGetErrorString(e));
}

constexpr int kMaxSmem = 227 * 1024;
constexpr int kDecodeRowsPerSplit = 128;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int check_layer(const kvm_layer* l) {
  if (!l) return fail(KVM_ERR_BAD_ARGUMENT, "layer is NULL");
  if (l->head_dim != 32 && l->head_dim != 64 && l->head_dim != 128)
    return fail(KVM_ERR_UNSUPPORTED, "head_dim %d not supported (32, 64 or 128; d_qk_head must equal d_v_head)", l->head_dim);
  if (l->n_kv_heads <= 0 || l->n_q_heads <= 0 || l->n_q_heads % l->n_kv_heads)
    return fail(KVM_ERR_BAD_ARGUMENT, "n_q_heads %d must be a positive multiple of n_kv_heads %d", l->n_q_heads, l->n_kv_heads);
  if (l->chunk_len < 16 || l->chunk_len % 16 || l->chunk_len > 512)
    return fail(KVM_ERR_UNSUPPORTED, "chunk_len %d must be a multiple of 16 in [16, 512]", l->chunk_len);
  if (l->n_bswa_chunks < 1) return fail(KVM_ERR_BAD_ARGUMENT, "n_bswa_chunks %d must be >= 1", l->n_bswa_chunks);
  if (l->rope_dim < 0 || l->rope_dim > l->head_dim)
    return fail(KVM_ERR_BAD_ARGUMENT, "rope_dim %d outside [0, head_dim]", l->rope_dim);
  if (l->sink_len < 0) return fail(KVM_ERR_BAD_ARGUMENT, "sink_len %d negative", l->sink_len);
  if (!l->ln_weight_dev || !l->ln_bias_dev || !l->front_temp_dev || !l->state_temp_dev)
    return fail(KVM_ERR_BAD_ARGUMENT, "layer parameter arrays must not be NULL");
  return KVM_OK;
}

LayerDev to_dev(const kvm_layer* l) {
  LayerDev L;
  L.Hq = l->n_q_heads; L.Hkv = l->n_kv_heads; L.C = l->chunk_len; L.W = l->n_bswa_chunks;
  L.rope_dim = l->rope_dim; L.sink_len = l->sink_len;
  L.gate_keys = l->gate_keys; L.gate_values = l->gate_values; L.gate_appends = l->gate_appends;
  L.gate_initial = l->gate_initial; L.ln_eps = l->ln_eps;
  L.ln_w = l->ln_weight_dev; L.ln_b = l->ln_bias_dev; L.front_temp = l->front_temp_dev; L.state_temp = l->state_temp_dev;
  return L;
}

Tensor4 to_dev(const kvm_tensor4& t) {
  Tensor4 r;
  r.ptr = static_cast<const bf16*>(t.ptr); r.sb = t.stride_b; r.sh = t.stride_h; r.st = t.stride_t;
  return r;
}

int check_tensor(const kvm_tensor4& t, const char* name, int row_elems) {
  if (!t.ptr) return fail(KVM_ERR_BAD_ARGUMENT, "%s is NULL", name);
  if (row_elems >= 8) {
    if (((uintptr_t)t.ptr) % 16 || t.stride_b % 8 || t.stride_h % 8 || t.stride_t % 8)
      return fail(KVM_ERR_BAD_ARGUMENT, "%s: base pointer and strides must be multiples of 16 bytes", name);
  }
  return KVM_OK;
}

MemoryDev to_dev(const kvm_memory& m) {
  MemoryDev r;
  r.k_sum = static_cast<bf16*>(m.k_sum); r.v_sum = static_cast<bf16*>(m.v_sum); r.vlen = m.vlen;
  r.k_attn = static_cast<bf16*>(m.k_attn); r.v_attn = static_cast<bf16*>(m.v_attn); r.capacity = m.capacity;
  return r;
}

int check_memory(const kvm_memory& m, const kvm_layer* l) {
  if (!m.k_sum || !m.v_sum || !m.vlen || !m.k_attn || !m.v_attn) return fail(KVM_ERR_BAD_ARGUMENT, "memory arrays must not be NULL");
  if (m.capacity <= 0) return fail(KVM_ERR_CAPACITY, "memory capacity %d must be positive", m.capacity);
  const size_t smem = update_smem_bytes(l->head_dim, l->chunk_len, m.capacity);
  if (smem > (size_t)kMaxSmem)
    return fail(KVM_ERR_CAPACITY, "memory capacity %d rows needs %zu bytes of shared memory for the update (limit %d)",
                m.capacity, smem, kMaxSmem);
  return KVM_OK;
}

// Prefill scratch: the row pool of the memory's attention view (every update writes at most C fresh
// rows per kv row), the per-version index tables, and the prepared-key scratch of the update variant
// that cannot stage a block in shared memory.
struct PrefillWs {
  size_t status, pool_k, pool_v, ver_idx, pk, pk_all, gk_all, route, born, tbits, total;
  long long pool_rows;
};
PrefillWs prefill_ws(const kvm_layer* l, int batch, long long seq_len, long long ver_rows) {
  const size_t rows = (size_t)batch * l->n_kv_heads;
  const size_t D = l->head_dim;
  const long long C = l->chunk_len;
  const long long n_qblocks = (seq_len + C - 1) / C;
  const long long n_plan = n_qblocks > l->n_bswa_chunks ? n_qblocks - l->n_bswa_chunks : 1;
  PrefillWs w;
  w.pool_rows = ver_rows > 0 ? C * n_plan : 0;
  size_t off = 0;
  w.status = off; off = 256;  // device status word written by kernels whose bounded waits expire
  w.pool_k = off; off = align_up(off + rows * (size_t)w.pool_rows * D * 2, 256);
  w.pool_v = off; off = align_up(off + rows * (size_t)w.pool_rows * D * 2, 256);
  w.ver_idx = off; off = align_up(off + rows * (size_t)ver_rows * 4, 256);
  w.pk = off; off = align_up(off + rows * (size_t)C * D * 2, 256);
  w.pk_all = off; off = align_up(off + (n_plan > 1 ? rows * (size_t)(n_plan * C) * D * 2 : 0), 256);  // prepared keys of all consumed tokens
  // gated keys of all consumed tokens and the routing decisions (the chain on the tensor cores reads its operands
  // from memory and hands the decisions to the value pass)
  const bool tc = D == 128 && (C == 128 || C == 256) && n_plan > 1;
  w.gk_all = off; off = align_up(off + (tc ? rows * (size_t)(n_plan * C) * D * 2 : 0), 256);
  w.route = off; off = align_up(off + (tc ? rows * (size_t)(n_plan * C) * 4 : 0), 256);
  // for the value side: the token that created each memory row (at most C * n_plan rows), one bit per (update, row)
  const size_t max_rows = (size_t)C * n_plan;
  w.born = off; off = align_up(off + (tc ? rows * max_rows * 4 : 0), 256);
  // (behind the bit table: control words of the value side, one progress flag per CTA of the routing kernel and a list
  // of up to 1024 jobs that spare CTAs of the routing's launch gave back)
  w.tbits = off; off = align_up(off + (tc ? rows * (size_t)n_plan * ((max_rows + 31) / 32) * 4 + (4 + rows * 8 + 1024) * 4 : 0), 256);
  w.total = off;
  return w;
}

struct DecodeWs {
  size_t pk, partial, counters, total;
  int nsplit_max;
};
DecodeWs decode_ws(const kvm_layer* l, int batch, int max_rows) {
  const size_t rows = (size_t)batch * l->n_kv_heads;
  const size_t D = l->head_dim;
  DecodeWs w;
  w.nsplit_max = (max_rows + kDecodeRowsPerSplit - 1) / kDecodeRowsPerSplit + 2;  // memory / window / wrapped window runs
  size_t off = 0;
  w.counters = off; off = align_up(off + (rows + batch + 1) * 4, 256);  // row counters, launch counter (+ spare), status word
  w.pk = off; off = align_up(off + rows * (size_t)l->chunk_len * D * 2, 256);
  w.partial = off; off = align_up(off + (size_t)batch * l->n_q_heads * w.nsplit_max * (D + 2) * 4, 256);
  w.total = off;
  return w;
}

// ---- scratch for kvm_decode_step_static: lives in the library image, one copy per GPU that loads it.
// In host code the name below is only a host-side handle of the symbol, never a device address: the
// address a kernel can use is looked up with cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[KVM_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "kvm_decode_step_static: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(KVM_ERR_UNSUPPORTED, "kvm_decode_step_static: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "kvm_decode_step_static: cudaGetSymbolAddress");
    if (!p) return fail(KVM_ERR_CUDA, "kvm_decode_step_static: symbol address is NULL");
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return KVM_OK;
}

}  // namespace

namespace kvm {
cudaError_t launch_prologue(int D, const LayerDev& L, const PrologueDev& p, int batch, long long T, cudaStream_t stream);
cudaError_t launch_interleave_shards(void* dst, const void* src, int n_shards, long long n_tokens, long long shard_bytes, cudaStream_t stream);
}
using kvm::launch_interleave_shards;

extern "C" {

const char* kvm_last_error_string(void) { return g_err; }

int kvm_abi_version(void) { return 100; }

size_t kvm_prefill_workspace_bytes(const kvm_layer* layer, int32_t batch, int64_t seq_len, int64_t total_version_rows) {
  if (!layer || batch <= 0 || total_version_rows < 0) return 0;
  return prefill_ws(layer, batch, seq_len, total_version_rows).total;
}

static int prefill_forward_impl(const kvm_layer* layer, int32_t batch, int64_t seq_len, kvm_tensor4 q, kvm_tensor4 k,
                                kvm_tensor4 v, kvm_tensor4 gate, const kvm_update_plan* plan_dev,
                                const kvm_update_plan* plan_host, int32_t n_updates, int64_t total_version_rows,
                                kvm_memory memory, void* out, int32_t* route_dev, void* workspace, size_t workspace_bytes,
                                uint32_t phases, void* stream, const kvm::GatherDst* gd) {
  g_err[0] = 0;
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0 || seq_len <= 0) return fail(KVM_ERR_BAD_ARGUMENT, "batch %d and seq_len %lld must be positive", batch, (long long)seq_len);
  if ((phases & 3u) == 0 || (phases & ~63u)) return fail(KVM_ERR_BAD_ARGUMENT, "phases %u must be a combination of KVM_PREFILL_CHAIN and KVM_PREFILL_ATTENTION", phases);
  const int D = layer->head_dim, C = layer->chunk_len, W = layer->n_bswa_chunks;
  if (int rc = check_tensor(q, "q", D)) return rc;
  if (int rc = check_tensor(k, "k", D)) return rc;
  if (int rc = check_tensor(v, "v", D)) return rc;
  if (int rc = check_tensor(gate, "gate", 1)) return rc;
  if (int rc = check_memory(memory, layer)) return rc;
  if (!plan_dev || !plan_host || !out) return fail(KVM_ERR_BAD_ARGUMENT, "plan and out must not be NULL");
  const long long n_qblocks = (seq_len + C - 1) / C;
  const long long want_plan = n_qblocks > W ? n_qblocks - W : 1;
  if (n_updates + 1 != want_plan)
    return fail(KVM_ERR_BAD_ARGUMENT, "plan has %d entries, seq_len %lld with block %d and window %d needs %lld", n_updates + 1,
                (long long)seq_len, C, W, want_plan);
  // the plan must be self-consistent and fit the buffers (no kernel is launched otherwise)
  long long S = 0, max_ver_end = 0;
  for (int u = 0; u <= n_updates; ++u) {
    const kvm_update_plan& p = plan_host[u];
    const long long expect_append_max = (u == 0) ? (seq_len < C ? seq_len : C) : C;
    if (p.state_before != S || p.n_append < 0 || p.n_append > expect_append_max || (u == 0 && p.n_append != expect_append_max))
      return fail(KVM_ERR_BAD_ARGUMENT, "plan entry %d inconsistent (state_before %d, n_append %d, expected state %lld)", u,
                  p.state_before, p.n_append, S);
    S += p.n_append;
    if (S > memory.capacity) return fail(KVM_ERR_CAPACITY, "plan entry %d grows the memory to %lld rows, capacity is %d", u, S, memory.capacity);
    if (u > 0 && S <= (layer->sink_len < S ? layer->sink_len : S) && p.n_append < C)
      return fail(KVM_ERR_BAD_ARGUMENT, "update %d merges into a memory with no non-sink row", u);
    if (n_qblocks > W && (phases & KVM_PREFILL_ATTENTION)) {
      if (p.version_row < 0) return fail(KVM_ERR_BAD_ARGUMENT, "plan entry %d: version_row %d must not be negative", u, p.version_row);
      if (p.version_row + S > max_ver_end) max_ver_end = p.version_row + S;
    }
  }
  if (max_ver_end > total_version_rows) return fail(KVM_ERR_CAPACITY, "versions need %lld rows, store has %lld", max_ver_end, (long long)total_version_rows);
  const PrefillWs ws = prefill_ws(layer, batch, seq_len, total_version_rows);
  if (!workspace || workspace_bytes < ws.total) return fail(KVM_ERR_CAPACITY, "workspace of %zu bytes given, %zu needed", workspace_bytes, ws.total);
  if (((uintptr_t)workspace) % 256 || ((uintptr_t)out) % 16) return fail(KVM_ERR_BAD_ARGUMENT, "workspace must be 256-byte aligned and out 16-byte aligned");

  unsigned char* wsb = static_cast<unsigned char*>(workspace);
  cudaError_t e = cudaSuccess;
  // the status word belongs to a whole prefill: the chain phase opens it, an attention-only call on the same
  // workspace adds to it (so that a timeout of the chain is still seen after the attention call)
  if (phases & KVM_PREFILL_CHAIN) e = cudaMemsetAsync(wsb + ws.status, 0, sizeof(int), static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kvm_prefill_forward: cudaMemsetAsync");
  e = prefill_dispatch(D, to_dev(layer), batch, seq_len, to_dev(q), to_dev(k), to_dev(v), to_dev(gate), plan_dev,
                                   n_updates + 1, total_version_rows, to_dev(memory), static_cast<bf16*>(out), route_dev,
                                   reinterpret_cast<bf16*>(wsb + ws.pool_k), reinterpret_cast<bf16*>(wsb + ws.pool_v),
                                   ws.pool_rows, reinterpret_cast<int*>(wsb + ws.ver_idx),
                                   reinterpret_cast<bf16*>(wsb + ws.pk), reinterpret_cast<bf16*>(wsb + ws.pk_all),
                                   reinterpret_cast<bf16*>(wsb + ws.gk_all), reinterpret_cast<int*>(wsb + ws.route),
                                   reinterpret_cast<int*>(wsb + ws.born), reinterpret_cast<unsigned*>(wsb + ws.tbits), (int)S,
                                   reinterpret_cast<int*>(wsb + ws.status), phases,
                                   static_cast<cudaStream_t>(stream), gd);
  if (e == cudaErrorNotSupported && gd)
    return fail(KVM_ERR_UNSUPPORTED, "kvm_prefill_forward_gathered needs the tensor-core attention kernel (head_dim 128, blocks of a multiple of 128 tokens)");
  if (e != cudaSuccess) return cuda_fail(e, "kvm_prefill_forward");
  return KVM_OK;
}

int kvm_prefill_forward(const kvm_layer* layer, int32_t batch, int64_t seq_len, kvm_tensor4 q, kvm_tensor4 k,
                        kvm_tensor4 v, kvm_tensor4 gate, const kvm_update_plan* plan_dev,
                        const kvm_update_plan* plan_host, int32_t n_updates, int64_t total_version_rows,
                        kvm_memory memory, void* out, int32_t* route_dev, void* workspace, size_t workspace_bytes,
                        uint32_t phases, void* stream) {
  return prefill_forward_impl(layer, batch, seq_len, q, k, v, gate, plan_dev, plan_host, n_updates, total_version_rows, memory, out,
                              route_dev, workspace, workspace_bytes, phases, stream, nullptr);
}

int kvm_prefill_forward_gathered(const kvm_layer* layer, int32_t batch, int64_t seq_len, kvm_tensor4 q, kvm_tensor4 k,
                                 kvm_tensor4 v, kvm_tensor4 gate, const kvm_update_plan* plan_dev,
                                 const kvm_update_plan* plan_host, int32_t n_updates, int64_t total_version_rows,
                                 kvm_memory memory, int32_t n_ranks, int32_t rank, void* const* out_bases,
                                 int32_t* route_dev, void* workspace, size_t workspace_bytes, uint32_t phases, void* stream) {
  g_err[0] = 0;
  if (n_ranks < 2 || n_ranks > 8 || rank < 0 || rank >= n_ranks || !out_bases)
    return fail(KVM_ERR_BAD_ARGUMENT, "kvm_prefill_forward_gathered: n_ranks %d must be 2..8, rank %d inside it, out_bases not NULL", n_ranks, rank);
  kvm::GatherDst gd = {};
  gd.n_ranks = n_ranks;
  gd.rank = rank;
  for (int r = 0; r < n_ranks; ++r) {
    if (!out_bases[r] || ((uintptr_t)out_bases[r]) % 16)
      return fail(KVM_ERR_BAD_ARGUMENT, "kvm_prefill_forward_gathered: output buffer of rank %d is NULL or not 16-byte aligned", r);
    gd.base[r] = out_bases[r];
  }
  if (layer && (layer->head_dim != 128 || layer->chunk_len % 128 != 0 || (phases & KVM_PREFILL_LEGACY_ATTENTION)))
    return fail(KVM_ERR_UNSUPPORTED, "kvm_prefill_forward_gathered needs the tensor-core attention kernel (head_dim 128, blocks of a multiple of 128 tokens)");
  return prefill_forward_impl(layer, batch, seq_len, q, k, v, gate, plan_dev, plan_host, n_updates, total_version_rows, memory,
                              out_bases[rank], route_dev, workspace, workspace_bytes, phases, stream, &gd);
}

int kvm_prologue_forward(const kvm_layer* layer, int32_t batch, int64_t seq_len, const kvm_prologue* in, void* q_out,
                         void* k_out, void* v_out, void* gate_out, int64_t total_version_rows, void* workspace,
                         size_t workspace_bytes, void* stream) {
  g_err[0] = 0;
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0 || seq_len <= 0) return fail(KVM_ERR_BAD_ARGUMENT, "batch %d and seq_len %lld must be positive", batch, (long long)seq_len);
  if (!in || !in->q_lin || !in->k_lin || !in->v_lin || !q_out || !k_out || !v_out || !gate_out)
    return fail(KVM_ERR_BAD_ARGUMENT, "kvm_prologue_forward: projections and outputs must not be NULL");
  const int D = layer->head_dim;
  if (D != 32 && D != 64 && D != 128) return fail(KVM_ERR_UNSUPPORTED, "kvm_prologue_forward: head_dim %d (supported: 32, 64, 128)", D);
  const int n_shift = (in->shift_q != nullptr) + (in->shift_k != nullptr) + (in->shift_v != nullptr);
  if (n_shift != 0 && n_shift != 3) return fail(KVM_ERR_BAD_ARGUMENT, "token-shift scales must be given for q, k and v or for none");
  const int n_ln = (in->ln_q_w != nullptr) + (in->ln_q_b != nullptr) + (in->ln_k_w != nullptr) + (in->ln_k_b != nullptr);
  if (n_ln != 0 && n_ln != 4) return fail(KVM_ERR_BAD_ARGUMENT, "LayerNorm weights and biases must be given for q and k or for neither");
  if ((in->cos == nullptr) != (in->sin == nullptr)) return fail(KVM_ERR_BAD_ARGUMENT, "cos and sin must both be given or both be NULL");
  if (in->cos && in->rope_stride_b != 0 && in->rope_stride_b != seq_len * D)
    return fail(KVM_ERR_BAD_ARGUMENT, "rope_stride_b %lld must be 0 or seq_len*head_dim", (long long)in->rope_stride_b);
  const void* aligned[] = {in->q_lin, in->k_lin, in->v_lin, in->shift_q, in->shift_k, in->shift_v, in->prev_q, in->prev_k, in->prev_v,
                           in->cos, in->sin, q_out, k_out, v_out, in->ln_q_w, in->ln_q_b, in->ln_k_w, in->ln_k_b,
                           layer->ln_weight_dev, layer->ln_bias_dev};
  for (const void* a : aligned)
    if (((uintptr_t)a) % 16) return fail(KVM_ERR_BAD_ARGUMENT, "kvm_prologue_forward: tensors must be 16-byte aligned");
  kvm::PrologueDev p = {};
  p.q_lin = static_cast<const bf16*>(in->q_lin);
  p.k_lin = static_cast<const bf16*>(in->k_lin);
  p.v_lin = static_cast<const bf16*>(in->v_lin);
  p.gate_lin = static_cast<const bf16*>(in->gate_lin);
  p.shift_q = static_cast<const bf16*>(in->shift_q);
  p.shift_k = static_cast<const bf16*>(in->shift_k);
  p.shift_v = static_cast<const bf16*>(in->shift_v);
  p.prev_q = static_cast<const bf16*>(in->prev_q);
  p.prev_k = static_cast<const bf16*>(in->prev_k);
  p.prev_v = static_cast<const bf16*>(in->prev_v);
  p.ln_q_w = in->ln_q_w;
  p.ln_q_b = in->ln_q_b;
  p.ln_k_w = in->ln_k_w;
  p.ln_k_b = in->ln_k_b;
  p.ln_qk_eps = in->ln_qk_eps;
  p.cos = static_cast<const bf16*>(in->cos);
  p.sin = static_cast<const bf16*>(in->sin);
  p.rope_stride_b = in->rope_stride_b;
  p.q_out = static_cast<bf16*>(q_out);
  p.k_out = static_cast<bf16*>(k_out);
  p.v_out = static_cast<bf16*>(v_out);
  p.gate_out = static_cast<bf16*>(gate_out);
  const long long C = layer->chunk_len;
  const long long n_qblocks = (seq_len + C - 1) / C;
  const long long n_plan = n_qblocks > layer->n_bswa_chunks ? n_qblocks - layer->n_bswa_chunks : 1;
  if (workspace && n_plan > 1) {
    const PrefillWs ws = prefill_ws(layer, batch, seq_len, total_version_rows);
    if (workspace_bytes < ws.total) return fail(KVM_ERR_CAPACITY, "workspace of %zu bytes given, %zu needed", workspace_bytes, ws.total);
    if (((uintptr_t)workspace) % 256) return fail(KVM_ERR_BAD_ARGUMENT, "workspace must be 256-byte aligned");
    unsigned char* wsb = static_cast<unsigned char*>(workspace);
    p.pk_all = reinterpret_cast<bf16*>(wsb + ws.pk_all);
    p.gk_all = ws.route > ws.gk_all ? reinterpret_cast<bf16*>(wsb + ws.gk_all) : nullptr;  // present for the tensor-core chain's shapes
    p.n_tok = n_plan * C;
  }
  const cudaError_t e = kvm::launch_prologue(D, to_dev(layer), p, batch, seq_len, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kvm_prologue_forward");
  return KVM_OK;
}

int kvm_prefill_workspace_layout(const kvm_layer* layer, int32_t batch, int64_t seq_len, int64_t total_version_rows,
                                 kvm_prefill_layout* out) {
  g_err[0] = 0;
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0 || seq_len <= 0 || total_version_rows < 0 || !out)
    return fail(KVM_ERR_BAD_ARGUMENT, "batch and seq_len must be positive, total_version_rows not negative, out not NULL");
  const PrefillWs ws = prefill_ws(layer, batch, seq_len, total_version_rows);
  out->status_offset = ws.status;
  out->pool_k_offset = ws.pool_k;
  out->pool_v_offset = ws.pool_v;
  out->version_table_offset = ws.ver_idx;
  out->prepared_keys_offset = ws.pk_all;
  out->gated_keys_offset = ws.gk_all;
  out->pool_rows = ws.pool_rows;
  out->total_bytes = ws.total;
  return KVM_OK;
}

int kvm_prefill_status(void* workspace, void* stream) {
  g_err[0] = 0;
  if (!workspace) return fail(KVM_ERR_BAD_ARGUMENT, "workspace is NULL");
  int st = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && st != 0) e = cudaMemsetAsync(workspace, 0, sizeof(int), s);  // reported once
  if (e != cudaSuccess) return cuda_fail(e, "kvm_prefill_status");
  if (st == KVM_ERR_DEVICE_TIMEOUT) return fail(st, "a bounded wait inside a prefill kernel expired (device-side timeout)");
  if (st != 0) return fail(st, "a prefill kernel reported status %d", st);
  return KVM_OK;
}

size_t kvm_decode_workspace_bytes(const kvm_layer* layer, int32_t batch, int32_t max_rows_per_seq) {
  if (!layer || batch <= 0 || max_rows_per_seq <= 0) return 0;
  return decode_ws(layer, batch, max_rows_per_seq).total;
}

static int decode_step_impl(const kvm_layer* layer, int32_t batch, const kvm_decode_cache& cache, kvm_tensor4 q, kvm_tensor4 k,
                            kvm_tensor4 v, kvm_tensor4 gate, const int32_t* n_append_dev, int32_t any_update, int32_t max_rows,
                            void* out, int32_t* route_dev, void* workspace, size_t workspace_bytes, void* stream,
                            int overlap, const char* who, bool clear_counters = false) {
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0) return fail(KVM_ERR_BAD_ARGUMENT, "batch %d must be positive", batch);
  const int D = layer->head_dim;
  if (int rc = check_tensor(q, "q", D)) return rc;
  if (int rc = check_tensor(k, "k", D)) return rc;
  if (int rc = check_tensor(v, "v", D)) return rc;
  if (int rc = check_tensor(gate, "gate", 1)) return rc;
  if (layer->n_q_heads / layer->n_kv_heads > 16)
    return fail(KVM_ERR_UNSUPPORTED, "decode supports at most 16 query heads per kv head, got %d", layer->n_q_heads / layer->n_kv_heads);
  if (int rc = check_memory(cache.memory, layer)) return rc;
  if (!cache.ring_k || !cache.ring_v || !cache.ring_gate || !cache.total_len || !cache.state_len)
    return fail(KVM_ERR_BAD_ARGUMENT, "decode cache arrays must not be NULL");
  if (any_update && !n_append_dev) return fail(KVM_ERR_BAD_ARGUMENT, "any_update set but n_append_dev is NULL");
  if (!out) return fail(KVM_ERR_BAD_ARGUMENT, "out is NULL");
  const int row_bound = cache.memory.capacity + layer->n_bswa_chunks * layer->chunk_len;
  if (max_rows <= 0 || max_rows > row_bound) return fail(KVM_ERR_BAD_ARGUMENT, "max_rows %d outside (0, capacity + window = %d]", max_rows, row_bound);
  const DecodeWs ws = decode_ws(layer, batch, max_rows);
  if (!workspace || workspace_bytes < ws.total) return fail(KVM_ERR_CAPACITY, "%s: scratch of %zu bytes available, %zu needed", who, workspace_bytes, ws.total);
  if (((uintptr_t)workspace) % 256) return fail(KVM_ERR_BAD_ARGUMENT, "workspace must be 256-byte aligned");

  DecodeCacheDev c;
  c.mem = to_dev(cache.memory);
  c.ring_k = static_cast<bf16*>(cache.ring_k); c.ring_v = static_cast<bf16*>(cache.ring_v);
  c.ring_g = static_cast<bf16*>(cache.ring_gate); c.total_len = cache.total_len; c.state_len = cache.state_len;
  unsigned char* wsb = static_cast<unsigned char*>(workspace);
  if (any_update < 0 || any_update > batch) any_update = batch;  // count unknown: no overlap
  cudaError_t e;
  if (clear_counters) {  // every argument has been checked: the first thing enqueued is the clearing of the counters
    e = cudaMemsetAsync(wsb + ws.counters, 0, ((size_t)batch * layer->n_kv_heads + batch + 1) * sizeof(int),
                        static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, who);
  }
  e = decode_dispatch(D, to_dev(layer), batch, c, to_dev(q), to_dev(k), to_dev(v), to_dev(gate), n_append_dev,
                                  any_update, max_rows, static_cast<bf16*>(out), route_dev,
                                  reinterpret_cast<bf16*>(wsb + ws.pk), reinterpret_cast<float*>(wsb + ws.partial),
                                  reinterpret_cast<int*>(wsb + ws.counters), ws.nsplit_max, overlap,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, who);
  return KVM_OK;
}

int kvm_decode_step(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache, kvm_tensor4 q, kvm_tensor4 k,
                    kvm_tensor4 v, kvm_tensor4 gate, const int32_t* n_append_dev, int32_t any_update, int32_t max_rows,
                    void* out, int32_t* route_dev, void* workspace, size_t workspace_bytes, void* stream) {
  g_err[0] = 0;
  return decode_step_impl(layer, batch, cache, q, k, v, gate, n_append_dev, any_update, max_rows, out, route_dev, workspace,
                          workspace_bytes, stream, 1, "kvm_decode_step");
}

int kvm_decode_run(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache, int32_t n_steps, kvm_tensor4 q,
                   kvm_tensor4 k, kvm_tensor4 v, kvm_tensor4 gate, int64_t q_step_stride, int64_t kv_step_stride,
                   int64_t gate_step_stride, const int32_t* n_append_dev, const int32_t* any_update_host,
                   const int32_t* max_rows_host, void* out, void* workspace, size_t workspace_bytes, void* stream) {
  g_err[0] = 0;
  if (n_steps <= 0 || !any_update_host || !max_rows_host)
    return fail(KVM_ERR_BAD_ARGUMENT, "n_steps must be positive and the per-step host arrays not NULL");
  if (!layer) return fail(KVM_ERR_BAD_ARGUMENT, "layer is NULL");
  if (q_step_stride % 8 || kv_step_stride % 8) return fail(KVM_ERR_BAD_ARGUMENT, "step strides must be multiples of 16 bytes");
  const size_t out_stride = (size_t)batch * layer->n_q_heads * layer->head_dim;
  for (int i = 0; i < n_steps; ++i) {
    kvm_tensor4 qi = q, ki = k, vi = v, gi = gate;
    qi.ptr = static_cast<const uint16_t*>(q.ptr) + (size_t)i * q_step_stride;
    ki.ptr = static_cast<const uint16_t*>(k.ptr) + (size_t)i * kv_step_stride;
    vi.ptr = static_cast<const uint16_t*>(v.ptr) + (size_t)i * kv_step_stride;
    gi.ptr = static_cast<const uint16_t*>(gate.ptr) + (size_t)i * gate_step_stride;
    const int upd = any_update_host[i];
    if (upd && !n_append_dev) return fail(KVM_ERR_BAD_ARGUMENT, "step %d updates the memory but n_append_dev is NULL", i);
    int rc = decode_step_impl(layer, batch, cache, qi, ki, vi, gi, upd ? n_append_dev + (size_t)i * batch : nullptr, upd,
                              max_rows_host[i], static_cast<uint16_t*>(out) + (size_t)i * out_stride, nullptr, workspace,
                              workspace_bytes, stream, 1, "kvm_decode_run");
    if (rc) return rc;
  }
  return KVM_OK;
}

int kvm_decode_step_static(const kvm_layer* layer, int32_t batch, kvm_decode_cache cache, kvm_tensor4 q, kvm_tensor4 k,
                           kvm_tensor4 v, kvm_tensor4 gate, const int32_t* n_append_dev, int32_t any_update,
                           int32_t max_rows, void* out, int32_t* route_dev, void* stream) {
  g_err[0] = 0;
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0 || max_rows <= 0) return fail(KVM_ERR_BAD_ARGUMENT, "batch %d and max_rows %d must be positive", batch, max_rows);
  const DecodeWs ws = decode_ws(layer, batch, max_rows);
  if (ws.total > (size_t)KVM_STATIC_SCRATCH_BYTES)
    return fail(KVM_ERR_CAPACITY,
                "kvm_decode_step_static: this shape needs %zu bytes of scratch, the built-in scratch holds %u "
                "(batch %d x %d kv heads, block %d, head_dim %d, %d rows); use kvm_decode_step with a caller workspace",
                ws.total, (unsigned)KVM_STATIC_SCRATCH_BYTES, batch, layer->n_kv_heads, layer->chunk_len, layer->head_dim, max_rows);
  void* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  // the array keeps whatever the previous call left: the split counters (and the status word behind them) must
  // start at zero; they are cleared on the stream once the remaining arguments have been validated
  return decode_step_impl(layer, batch, cache, q, k, v, gate, n_append_dev, any_update, max_rows, out, route_dev, scratch,
                          (size_t)KVM_STATIC_SCRATCH_BYTES, stream, 0, "kvm_decode_step_static", true);
}

int kvm_decode_status(const kvm_layer* layer, int32_t batch, void* workspace, void* stream) {
  g_err[0] = 0;
  if (!layer || batch <= 0 || layer->n_kv_heads <= 0) return fail(KVM_ERR_BAD_ARGUMENT, "layer is NULL or batch %d not positive", batch);
  if (!workspace) {  // the built-in scratch of kvm_decode_step_static
    if (int rc = static_scratch_for_current_device(&workspace)) return rc;
  }
  int* word = reinterpret_cast<int*>(static_cast<unsigned char*>(workspace)) + (size_t)batch * layer->n_kv_heads + batch;
  int st = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&st, word, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && st != 0) e = cudaMemsetAsync(word, 0, sizeof(int), s);  // reported once
  if (e != cudaSuccess) return cuda_fail(e, "kvm_decode_status");
  if (st == KVM_ERR_DEVICE_TIMEOUT) return fail(st, "a bounded wait inside a decode kernel expired (device-side timeout)");
  if (st != 0) return fail(st, "a decode kernel reported status %d", st);
  return KVM_OK;
}

int kvm_memory_refresh(const kvm_layer* layer, int32_t batch, kvm_memory memory, const int32_t* state_len_dev, void* stream) {
  g_err[0] = 0;
  if (int rc = check_layer(layer)) return rc;
  if (batch <= 0 || !state_len_dev) return fail(KVM_ERR_BAD_ARGUMENT, "batch must be positive and state_len_dev not NULL");
  if (!memory.k_sum || !memory.v_sum || !memory.vlen || !memory.k_attn || !memory.v_attn || memory.capacity <= 0)
    return fail(KVM_ERR_BAD_ARGUMENT, "memory arrays must not be NULL");
  cudaError_t e = refresh_dispatch(layer->head_dim, to_dev(layer), batch, to_dev(memory), state_len_dev, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kvm_memory_refresh");
  return KVM_OK;
}

int kvm_interleave_shards(void* dst, const void* src, int32_t n_shards, int64_t n_tokens, int64_t shard_bytes, void* stream) {
  g_err[0] = 0;
  if (!dst || !src || n_shards <= 0 || n_tokens <= 0 || shard_bytes <= 0 || shard_bytes % 16 || ((uintptr_t)dst) % 16 || ((uintptr_t)src) % 16)
    return fail(KVM_ERR_BAD_ARGUMENT, "kvm_interleave_shards: buffers must be 16-byte aligned and shard_bytes (%lld) a positive multiple of 16",
                (long long)shard_bytes);
  cudaError_t e = launch_interleave_shards(dst, src, n_shards, n_tokens, shard_bytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "kvm_interleave_shards");
  return KVM_OK;
}

}  // extern "C"
