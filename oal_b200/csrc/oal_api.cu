// C ABI of oal_b200: argument checking, workspace carving and kernel sequencing.
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, const char* detail = "") {
  snprintf(g_error, sizeof(g_error), fmt, detail);
  return code;
}

int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_error, sizeof(g_error), "%s: %s", where, cudaGetErrorString(e));
  return OAL_ERR_CUDA;
}

// ---- launch accounting and optional per-kernel timing -----------------------------------
// Counterpart of the reference's opt-in stage profiler (oal_attention/hd_block_gemm_profiling.py):
// a launch counter that is always on, and CUDA-event pairs around every launch when enabled.
struct ProfEntry {
  const char* name;
  cudaEvent_t start, stop;
};
std::mutex g_prof_mutex;
std::vector<ProfEntry> g_prof_entries;
std::atomic<int> g_prof_enabled{0};
std::atomic<long long> g_launches{0};

struct LaunchScope {
  cudaStream_t st;
  bool timed = false;
  ProfEntry entry{};
  // `timing`: false for entry points that promise to make no allocating call (event creation is one)
  LaunchScope(const char* name, cudaStream_t stream, int launches = 1, bool timing = true) : st(stream) {
    g_launches += launches;
    if (!timing || !g_prof_enabled.load()) return;
    entry.name = name;
    if (cudaEventCreate(&entry.start) != cudaSuccess || cudaEventCreate(&entry.stop) != cudaSuccess) return;
    timed = true;
    cudaEventRecord(entry.start, st);
  }
  ~LaunchScope() {
    if (!timed) return;
    cudaEventRecord(entry.stop, st);
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    g_prof_entries.push_back(entry);
  }
};

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

// ---- deferred status words ------------------------------------------------------------------
// A ring of pinned host words per device, filled by 4-byte copies on a stream of the library's own: the
// copy never sits on the caller's stream (where it would queue behind the application's own device-to-host
// copies and hold the kernels after it), and queueing one costs two event records and a copy instead of
// the tensor, stream and event objects a Python implementation creates per call.
constexpr int STATUS_RING = 1024;
struct StatusRing {
  cudaStream_t stream = nullptr;
  int32_t* host = nullptr;
  cudaEvent_t ready[STATUS_RING] = {};
  cudaEvent_t done[STATUS_RING] = {};
  long long next = 0;
};
std::mutex g_status_mutex;
StatusRing g_status[64];

// ---- side streams ------------------------------------------------------------------------------
// Small kernels that nothing on the main chain waits for (the per-head factor table of the forward, the
// coefficient-gradient reductions, the reverse state scan and the whole key/value chain of the backward)
// run on two library-owned streams, forked from and joined back into the caller's stream with events, so
// every entry point still looks like work on one stream from outside (and can be captured as such).
// Streams and events are created once per device, on first use; oal_set_overlap(0) keeps everything on
// the caller's stream (the per-kernel timing of the profile report is only meaningful that way).
std::atomic<int> g_overlap{1};
struct SideStreams {
  cudaStream_t s[2] = {nullptr, nullptr};
  cudaEvent_t fork = nullptr, join[2] = {nullptr, nullptr};
  bool ok = false;
};
std::mutex g_side_mutex;
SideStreams g_side[64];

SideStreams* side_streams() {
  if (!g_overlap.load()) return nullptr;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideStreams& x = g_side[dev];
  if (!x.ok) {
    bool good = cudaEventCreateWithFlags(&x.fork, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 2 && good; ++i)
      good = cudaStreamCreateWithFlags(&x.s[i], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&x.join[i], cudaEventDisableTiming) == cudaSuccess;
    if (!good) return nullptr;
    x.ok = true;
  }
  return &x;
}
// side stream i starts after everything queued on `st` so far
cudaStream_t fork_to(SideStreams* x, int i, cudaStream_t st) {
  if (!x) return st;
  if (cudaEventRecord(x->fork, st) != cudaSuccess || cudaStreamWaitEvent(x->s[i], x->fork, 0) != cudaSuccess) return st;
  return x->s[i];
}
// mark the end of what was queued on side stream i; `st` waits for that mark in join_wait
void join_mark(SideStreams* x, int i, cudaStream_t side, cudaStream_t st) {
  if (x && side != st) cudaEventRecord(x->join[i], side);
}
void join_wait(SideStreams* x, int i, cudaStream_t side, cudaStream_t st) {
  if (x && side != st) cudaStreamWaitEvent(st, x->join[i], 0);
}

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <class T>
  T* take(size_t count) {
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += align_up(count * sizeof(T));
    return p;
  }
};

int check_problem(const OalProblem* p) {
  if (!p) return fail(OAL_ERR_ARGUMENT, "problem is NULL");
  if (p->batch < 1 || p->q_heads < 1 || p->kv_heads < 1 || p->seq_len < 1)
    return fail(OAL_ERR_ARGUMENT, "batch, head counts and seq_len must be positive");
  if (p->q_heads % p->kv_heads) return fail(OAL_ERR_ARGUMENT, "q_heads must be divisible by kv_heads");
  if (p->head_dim != OAL_HEAD_DIM || p->value_dim != OAL_HEAD_DIM)
    return fail(OAL_ERR_ARGUMENT, "head_dim and value_dim must be 64 (the host pads smaller heads)");
  if (p->groups < 1 || p->groups > OAL_MAX_GROUPS)
    return fail(OAL_ERR_ARGUMENT, "groups must be in 1..16");
  if (p->io_dtype < 0 || p->io_dtype > 2 || p->out_dtype < 0 || p->out_dtype > 2)
    return fail(OAL_ERR_DTYPE, "io_dtype / out_dtype must be fp32, bf16 or fp16");
  if (p->precision != OAL_PRECISION_FP32_IEEE && p->precision != OAL_PRECISION_BF16_TENSORCORE)
    return fail(OAL_ERR_DTYPE, "unknown precision mode");
  if (p->precision == OAL_PRECISION_BF16_TENSORCORE) {
    if (p->io_dtype != OAL_DTYPE_BF16) return fail(OAL_ERR_DTYPE, "bf16_tensorcore requires bf16 q, k, v");
    if (p->chunk != 128) return fail(OAL_ERR_ARGUMENT, "bf16_tensorcore requires chunk == 128");
  }
  if (!(p->floor > 0.f)) return fail(OAL_ERR_ARGUMENT, "floor must be positive");
  if (p->flags & ~OAL_FLAG_OUT_TOKEN_MAJOR) return fail(OAL_ERR_ARGUMENT, "unknown bits in flags");
  if ((p->flags & OAL_FLAG_OUT_TOKEN_MAJOR) &&
      (p->precision != OAL_PRECISION_BF16_TENSORCORE || p->groups + 1 > oal::intra_coef_terms()))
    return fail(OAL_ERR_ARGUMENT, "token-major out needs bf16_tensorcore and at most 8 groups per head");
  return OAL_OK;
}

struct BackwardSpace {
  float* g;
  float* coef_pairs;
  size_t bytes;
};

BackwardSpace carve_backward(const OalProblem* p, void* ws) {
  Carver c(ws);
  BackwardSpace s;
  const size_t rows = (size_t)p->batch * p->q_heads * p->seq_len;
  s.g = c.take<float>(rows * oal::EP);
  s.coef_pairs = c.take<float>((size_t)p->batch * p->q_heads * oal::pairs_tiles(p->seq_len) * oal::NCOEF);
  s.bytes = c.off;
  return s;
}

constexpr int kChunk = 128;

int chunk_count(const OalProblem* p) { return (p->seq_len + kChunk - 1) / kChunk; }

struct ForwardSpaceTC {
  float* coef_table;
  float* ds;
  size_t bytes;
};

// the intra-chunk term runs on the tensor cores for heads with at most 8 groups (else token-pair kernels)
bool tc_intra(const OalProblem* p) { return p->groups + 1 <= oal::intra_coef_terms(); }

int make_head_factors(const OalProblem* p, const int32_t* dim_perm, const int32_t* group_start, const float* coef_a,
                      const float* coef_b, const float* coef_c, void* factors, cudaStream_t st, bool timing = true) {
  LaunchScope scope("head_factors", st, 1, timing);
  cudaError_t e = oal::build_head_factors(dim_perm, group_start, coef_a, coef_b, coef_c, p->q_heads, p->groups,
                                          p->scale, factors, st);
  return e == cudaSuccess ? OAL_OK : fail_cuda(e, "head factor kernel");
}

ForwardSpaceTC carve_forward_tc(const OalProblem* p, void* ws) {
  Carver c(ws);
  ForwardSpaceTC s;
  const size_t units = (size_t)p->batch * p->kv_heads;
  s.coef_table = c.take<float>((size_t)p->q_heads * oal::state_rows());
  s.ds = c.take<float>(units * chunk_count(p) * oal::state_rows() * oal::EP);
  s.bytes = c.off;
  return s;
}

// The buffer the forward hands to the backward: the bf16 carry images of every chunk (the MMA operand),
// the images of their rounding remainders (read only by the coefficient-gradient dot products), then the
// per-head factor table of the intra-chunk kernels (the backward of the same call sees the same
// coefficients, so it does not factor them again).
size_t saved_images_bytes_tc(const OalProblem* p) {
  return align_up((size_t)p->batch * p->kv_heads * chunk_count(p) * oal::state_image_bytes_per_chunk());
}
size_t saved_state_bytes_tc(const OalProblem* p) { return 2 * saved_images_bytes_tc(p) + oal::head_factor_bytes(p->q_heads); }
void* saved_remainders(const OalProblem* p, const void* saved_state) {
  return const_cast<char*>(static_cast<const char*>(saved_state)) + saved_images_bytes_tc(p);
}
void* saved_factors(const OalProblem* p, const void* saved_state) {
  return const_cast<char*>(static_cast<const char*>(saved_state)) + 2 * saved_images_bytes_tc(p);
}

struct BackwardSpaceTC {
  float* g;
  float* coef_pairs;
  void* gimg;
  float* coef_table;
  float* dcarry;
  void* dt_img;
  float* dcoef_partial;
  float* dcoef;
  float* slots;
  float *dq_cross, *dk_cross, *dv_cross;
  float *dk_part, *dv_part;      // per-query-head intra-chunk shares of dk / dv
  size_t bytes;
};

BackwardSpaceTC carve_backward_tc(const OalProblem* p, void* ws) {
  Carver c(ws);
  BackwardSpaceTC s;
  const size_t units = (size_t)p->batch * p->kv_heads, nb = chunk_count(p);
  const size_t qrows = (size_t)p->batch * p->q_heads * p->seq_len;
  const size_t krows = (size_t)p->batch * p->kv_heads * p->seq_len;
  const size_t slab_image = oal::state_slab_image_bytes();
  s.g = c.take<float>(qrows * oal::EP);
  s.coef_pairs = c.take<float>((size_t)p->batch * p->q_heads * oal::pairs_tiles(p->seq_len) * oal::NCOEF);
  s.gimg = c.take<char>(2 * (size_t)p->batch * p->q_heads * nb * slab_image);   // hi image, then lo image
  s.coef_table = c.take<float>((size_t)p->q_heads * oal::state_rows());
  s.dcarry = c.take<float>(units * nb * oal::state_rows() * oal::EP);
  s.dt_img = c.take<char>(units * nb * oal::state_image_bytes_per_chunk());
  s.dcoef_partial = c.take<float>(2 * (size_t)p->batch * nb * p->q_heads * oal::state_rows());   // two column halves
  s.dcoef = c.take<float>((size_t)p->q_heads * oal::state_rows());
  s.slots = c.take<float>((size_t)p->q_heads * oal::NCOEF);
  s.dq_cross = c.take<float>(qrows * oal::HD);
  s.dk_cross = c.take<float>(krows * oal::HD);
  s.dv_cross = c.take<float>(krows * oal::VD);
  s.dk_part = c.take<float>(qrows * oal::HD);
  s.dv_part = c.take<float>(qrows * oal::VD);
  s.bytes = c.off;
  return s;
}

// Stage A of the tensor-core backward: everything that does not depend on later tokens' state
// gradient (normalisation VJP, coefficient table, per-chunk dCarry and coefficient partial sums).
int backward_state_stage(const OalProblem* p, const void* q, const int32_t* dim_perm, const int32_t* group_start,
                         const float* coef_a, const float* coef_b, const float* coef_c, const float* num,
                         const float* den, const void* saved_state, const void* grad_out, const float* grad_num,
                         const float* grad_den, const BackwardSpaceTC& s, int32_t* status, cudaStream_t st) {
  const int nb = chunk_count(p);
  const int mask = p->grad_mask;
  const bool want_c = mask & OAL_GRAD_COEF;
  cudaError_t e;
  { LaunchScope scope("norm_vjp", st);
    // the fp32 rows of g are read by the token-pair kernels only (heads with more than 8 groups)
    e = oal::norm_vjp_image(grad_out, p->out_dtype, grad_num, grad_den, num, den, p->floor,
                            tc_intra(p) ? nullptr : s.g, s.gimg,
                            p->batch * p->q_heads, p->seq_len, nb,
                            (p->flags & OAL_FLAG_OUT_TOKEN_MAJOR) ? p->q_heads : 0, st); }
  if (e != cudaSuccess) return fail_cuda(e, "normalisation VJP kernel");
  { LaunchScope scope("coef_table", st);
    e = oal::build_coef_table(dim_perm, group_start, coef_a, coef_b, coef_c, p->q_heads, p->groups, p->scale, s.coef_table, st); }
  if (e != cudaSuccess) return fail_cuda(e, "coefficient table kernel");
  if (mask & (OAL_GRAD_K | OAL_GRAD_V | OAL_GRAD_COEF)) {
    { LaunchScope scope("dstate_heads", st);
      e = oal::dstate_heads(q, s.gimg, want_c ? saved_state : nullptr, want_c ? saved_remainders(p, saved_state) : nullptr,
                            s.coef_table, s.dcarry,
                            want_c ? s.dcoef_partial : nullptr, p->batch, p->q_heads, p->kv_heads, p->seq_len, nb,
                            p->scale, status, st); }
    if (e != cudaSuccess) return fail_cuda(e, "state gradient kernel");
  }
  return OAL_OK;
}

oal::PairArgs base_args(const OalProblem* p, const void* q, const void* k, const void* v,
                        const int32_t* perm, const int32_t* gstart, const float* A, const float* B,
                        const float* C, int32_t* status) {
  oal::PairArgs a;
  memset(&a, 0, sizeof(a));
  a.B = p->batch; a.Hq = p->q_heads; a.Hkv = p->kv_heads; a.N = p->seq_len; a.G = p->groups;
  a.window = 0;
  a.io_dt = p->io_dtype; a.out_dt = p->out_dtype;
  a.scale = p->scale; a.floor = p->floor;
  a.q = q; a.k = k; a.v = v;
  a.dim_perm = perm; a.group_start = gstart;
  a.A = A; a.Bc = B; a.Cc = C;
  a.status = status;
  return a;
}

}  // namespace

extern "C" {

int oal_rope_pack(const void* q_flat, const void* k_flat, const void* v_flat, const float* cosv, const float* sinv,
                  void* q, void* k, void* v, int batch, int seq_len, int q_heads, int kv_heads, void* stream) {
  if (batch < 0 || seq_len < 0 || q_heads < 1 || kv_heads < 1) return fail(OAL_ERR_ARGUMENT, "oal_rope_pack: bad geometry");
  if ((q_flat || k_flat) && (!cosv || !sinv)) return fail(OAL_ERR_ARGUMENT, "oal_rope_pack: cos / sin are required");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  LaunchScope scope("rope_pack", st, (q_flat ? 1 : 0) + (k_flat ? 1 : 0) + (v_flat ? 1 : 0));
  if (q_flat && (e = oal::rope_to_heads(q_flat, q, cosv, sinv, batch, seq_len, q_heads, true, st)) != cudaSuccess)
    return fail_cuda(e, "rotary pack kernel (q)");
  if (k_flat && (e = oal::rope_to_heads(k_flat, k, cosv, sinv, batch, seq_len, kv_heads, true, st)) != cudaSuccess)
    return fail_cuda(e, "rotary pack kernel (k)");
  if (v_flat && (e = oal::rope_to_heads(v_flat, v, nullptr, nullptr, batch, seq_len, kv_heads, false, st)) != cudaSuccess)
    return fail_cuda(e, "pack kernel (v)");
  return OAL_OK;
}

int oal_rope_unpack_grad(const void* dq, const void* dk, const void* dv, const float* cosv, const float* sinv,
                         void* dq_flat, void* dk_flat, void* dv_flat, int batch, int seq_len, int q_heads,
                         int kv_heads, void* stream) {
  if (batch < 0 || seq_len < 0 || q_heads < 1 || kv_heads < 1)
    return fail(OAL_ERR_ARGUMENT, "oal_rope_unpack_grad: bad geometry");
  if ((dq || dk) && (!cosv || !sinv)) return fail(OAL_ERR_ARGUMENT, "oal_rope_unpack_grad: cos / sin are required");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  LaunchScope scope("rope_unpack_grad", st, (dq ? 1 : 0) + (dk ? 1 : 0) + (dv ? 1 : 0));
  if (dq && (e = oal::rope_to_flat(dq, dq_flat, cosv, sinv, batch, seq_len, q_heads, true, st)) != cudaSuccess)
    return fail_cuda(e, "rotary unpack kernel (dq)");
  if (dk && (e = oal::rope_to_flat(dk, dk_flat, cosv, sinv, batch, seq_len, kv_heads, true, st)) != cudaSuccess)
    return fail_cuda(e, "rotary unpack kernel (dk)");
  if (dv && (e = oal::rope_to_flat(dv, dv_flat, nullptr, nullptr, batch, seq_len, kv_heads, false, st)) != cudaSuccess)
    return fail_cuda(e, "unpack kernel (dv)");
  return OAL_OK;
}

const char* oal_last_error_string(void) { return g_error; }

const char* oal_version_string(void) { return "oal_b200 0.1 sm_100a"; }

int64_t oal_launch_count(void) { return g_launches.load(); }

void oal_profile_enable(int enable) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  for (auto& e : g_prof_entries) {
    cudaEventDestroy(e.start);
    cudaEventDestroy(e.stop);
  }
  g_prof_entries.clear();
  g_prof_enabled.store(enable ? 1 : 0);
}

int oal_profile_report(char* buffer, size_t capacity) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  std::map<std::string, std::pair<int, double>> agg;
  for (auto& e : g_prof_entries) {
    if (cudaEventSynchronize(e.stop) != cudaSuccess) return fail(OAL_ERR_CUDA, "oal_profile_report: event synchronise failed");
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e.start, e.stop);
    auto& slot = agg[e.name];
    slot.first += 1;
    slot.second += ms;
    cudaEventDestroy(e.start);
    cudaEventDestroy(e.stop);
  }
  g_prof_entries.clear();
  std::string out = "{";
  bool first = true;
  for (auto& kv : agg) {
    char item[160];
    snprintf(item, sizeof(item), "%s\"%s\": [%d, %.6f]", first ? "" : ", ", kv.first.c_str(), kv.second.first,
             kv.second.second);
    out += item;
    first = false;
  }
  out += "}";
  if (!buffer || out.size() + 1 > capacity) return fail(OAL_ERR_ARGUMENT, "oal_profile_report: buffer too small");
  memcpy(buffer, out.c_str(), out.size() + 1);
  return OAL_OK;
}

int64_t oal_workspace_bytes(const OalProblem* p, int phase) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (phase < 0 || phase > 2) return fail(OAL_ERR_ARGUMENT, "phase must be 0 (forward), 1 (backward) or 2 (saved state)");
  if (p->precision == OAL_PRECISION_FP32_IEEE) {
    if (phase == 1) return (int64_t)carve_backward(p, nullptr).bytes;
    return 0;
  }
  if (phase == 0) return (int64_t)carve_forward_tc(p, nullptr).bytes;
  if (phase == 2) return (int64_t)saved_state_bytes_tc(p);
  return (int64_t)carve_backward_tc(p, nullptr).bytes;
}

int oal_forward(const OalProblem* p, const void* q, const void* k, const void* v, const int32_t* dim_perm,
                const int32_t* group_start, const float* coef_a, const float* coef_b, const float* coef_c,
                void* out, float* num, float* den, void* saved_state, const float* state_in,
                void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (!q || !k || !v || !dim_perm || !group_start || !coef_a || !coef_b || !coef_c || !out || !num || !den || !status)
    return fail(OAL_ERR_ARGUMENT, "oal_forward: NULL tensor pointer");
  (void)saved_state; (void)workspace; (void)workspace_bytes;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->precision == OAL_PRECISION_FP32_IEEE) {
    if (state_in) return fail(OAL_ERR_ARGUMENT, "fp32_ieee mode keeps no chunk state: state_in must be NULL");
    oal::PairArgs a = base_args(p, q, k, v, dim_perm, group_start, coef_a, coef_b, coef_c, status);
    a.out = out; a.num = num; a.den = den; a.accumulate = 0;
    cudaError_t e;
    { LaunchScope scope("pairs_forward", st); e = oal::pairs_forward(a, st); }
    if (e != cudaSuccess) return fail_cuda(e, "forward pair kernel");
    return OAL_OK;
  }
  // bf16_tensorcore: chunk states on the tensor cores, intra-chunk term from token pairs
  ForwardSpaceTC s = carve_forward_tc(p, workspace);
  if (!workspace || workspace_bytes < s.bytes) return fail(OAL_ERR_WORKSPACE, "oal_forward: workspace too small");
  if (!saved_state) return fail(OAL_ERR_ARGUMENT, "oal_forward: saved_state is NULL");
  const int units = p->batch * p->kv_heads, nb = chunk_count(p);
  cudaError_t e;
  // the factor table is needed by the last kernel only: it is computed beside the state kernels
  SideStreams* side = tc_intra(p) ? side_streams() : nullptr;
  void* factors = saved_factors(p, saved_state);
  cudaStream_t s0 = st;
  if (tc_intra(p)) {
    s0 = fork_to(side, 0, st);
    if (int rc2 = make_head_factors(p, dim_perm, group_start, coef_a, coef_b, coef_c, factors, s0)) return rc2;
    join_mark(side, 0, s0, st);
  }
  { LaunchScope scope("coef_table", st);
    e = oal::build_coef_table(dim_perm, group_start, coef_a, coef_b, coef_c, p->q_heads, p->groups, p->scale, s.coef_table, st); }
  if (e != cudaSuccess) return fail_cuda(e, "coefficient table kernel");
  if (!(p->grad_mask & OAL_GRAD_REUSE_STATE_STAGE)) {      // else: left in this workspace by oal_forward_local_state
    { LaunchScope scope("state_update", st); e = oal::state_update(k, v, s.ds, units, p->seq_len, nb, status, st); }
    if (e != cudaSuccess) return fail_cuda(e, "state update kernel");
  }
  { LaunchScope scope("state_scan", st); e = oal::state_scan(s.ds, saved_state, saved_remainders(p, saved_state), state_in, nullptr, units, nb, 0, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state scan kernel");
  { LaunchScope scope("cross_read_q", st);
    e = oal::cross_read(true, q, saved_state, s.coef_table, num, den, p->batch, p->q_heads,
                        p->q_heads / p->kv_heads, p->seq_len, nb, status, st); }
  if (e != cudaSuccess) return fail_cuda(e, "cross read kernel");
  if (tc_intra(p)) {
    join_wait(side, 0, s0, st);
    { LaunchScope scope("intra_forward", st);
      e = oal::intra_forward(q, k, v, factors, out, num, den, status, p->batch, p->q_heads, p->kv_heads, p->seq_len, nb,
                             p->out_dtype, p->floor, (p->flags & OAL_FLAG_OUT_TOKEN_MAJOR) != 0, st); }
    if (e != cudaSuccess) return fail_cuda(e, "intra-chunk forward kernel");
    return OAL_OK;
  }
  oal::PairArgs a = base_args(p, q, k, v, dim_perm, group_start, coef_a, coef_b, coef_c, status);
  a.window = kChunk;
  a.out = out; a.num = num; a.den = den; a.accumulate = 1;
  { LaunchScope scope("pairs_forward", st); e = oal::pairs_forward(a, st); }
  if (e != cudaSuccess) return fail_cuda(e, "forward pair kernel");
  return OAL_OK;
}

void oal_set_overlap(int enable) { g_overlap.store(enable ? 1 : 0); }

int oal_status_defer(const int32_t* status, void* stream, int64_t* ticket) {
  if (!status || !ticket) return fail(OAL_ERR_ARGUMENT, "oal_status_defer: NULL pointer");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "oal_status_defer");
  if (dev < 0 || dev >= 64) return fail(OAL_ERR_ARGUMENT, "oal_status_defer: device index out of range");
  std::lock_guard<std::mutex> lock(g_status_mutex);
  StatusRing& r = g_status[dev];
  if (!r.stream) {
    if ((e = cudaStreamCreateWithFlags(&r.stream, cudaStreamNonBlocking)) != cudaSuccess) return fail_cuda(e, "oal_status_defer");
    if ((e = cudaHostAlloc(reinterpret_cast<void**>(&r.host), STATUS_RING * sizeof(int32_t), cudaHostAllocPortable)) !=
        cudaSuccess)
      return fail_cuda(e, "oal_status_defer");
  }
  const int slot = (int)(r.next % STATUS_RING);
  if (!r.done[slot]) {
    if ((e = cudaEventCreateWithFlags(&r.ready[slot], cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&r.done[slot], cudaEventDisableTiming)) != cudaSuccess)
      return fail_cuda(e, "oal_status_defer");
  } else if ((e = cudaEventSynchronize(r.done[slot])) != cudaSuccess) {   // the slot's previous copy (1024 calls ago)
    return fail_cuda(e, "oal_status_defer");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((e = cudaEventRecord(r.ready[slot], st)) != cudaSuccess || (e = cudaStreamWaitEvent(r.stream, r.ready[slot], 0)) != cudaSuccess ||
      (e = cudaMemcpyAsync(r.host + slot, status, sizeof(int32_t), cudaMemcpyDeviceToHost, r.stream)) != cudaSuccess ||
      (e = cudaEventRecord(r.done[slot], r.stream)) != cudaSuccess)
    return fail_cuda(e, "oal_status_defer");
  *ticket = ((int64_t)dev << 48) | (int64_t)r.next;
  ++r.next;
  return OAL_OK;
}

int oal_status_poll(int64_t ticket, int block, int32_t* value) {
  if (!value) return fail(OAL_ERR_ARGUMENT, "oal_status_poll: NULL pointer");
  const int dev = (int)(ticket >> 48);
  const long long seq = (long long)(ticket & (((int64_t)1 << 48) - 1));
  if (dev < 0 || dev >= 64) return fail(OAL_ERR_ARGUMENT, "oal_status_poll: bad ticket");
  cudaEvent_t done;
  int32_t* word;
  {
    std::lock_guard<std::mutex> lock(g_status_mutex);
    StatusRing& r = g_status[dev];
    if (seq >= r.next || seq + STATUS_RING <= r.next) return fail(OAL_ERR_ARGUMENT, "oal_status_poll: ticket expired or unknown");
    done = r.done[seq % STATUS_RING];
    word = r.host + seq % STATUS_RING;
  }
  if (block) {
    cudaError_t e = cudaEventSynchronize(done);
    if (e != cudaSuccess) return fail_cuda(e, "oal_status_poll");
  } else {
    cudaError_t e = cudaEventQuery(done);
    if (e == cudaErrorNotReady) return 0;
    if (e != cudaSuccess) return fail_cuda(e, "oal_status_poll");
  }
  *value = *static_cast<volatile int32_t*>(word);
  return 1;
}

int oal_expand_factor(const float* factor, int factor_rows, int q_heads, int groups, float kernel_eps, float* coef_a,
                      float* coef_b, float* coef_c, void* stream) {
  if (!factor || !coef_a || !coef_b || !coef_c) return fail(OAL_ERR_ARGUMENT, "oal_expand_factor: NULL pointer");
  if (q_heads < 1 || groups < 1 || groups > OAL_MAX_GROUPS || (factor_rows != 1 && factor_rows != q_heads))
    return fail(OAL_ERR_ARGUMENT, "oal_expand_factor: bad geometry");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LaunchScope scope("expand_factor", st);
  cudaError_t e = oal::expand_factor(factor, factor_rows, q_heads, groups, kernel_eps, coef_a, coef_b, coef_c, st);
  return e == cudaSuccess ? OAL_OK : fail_cuda(e, "oal_expand_factor");
}

int oal_expand_factor_grad(const float* factor, int factor_rows, int q_heads, int groups, const float* d_coef_a,
                           const float* d_coef_b, const float* d_coef_c, float* d_factor, void* stream) {
  if (!factor || !d_coef_a || !d_coef_b || !d_coef_c || !d_factor)
    return fail(OAL_ERR_ARGUMENT, "oal_expand_factor_grad: NULL pointer");
  if (q_heads < 1 || groups < 1 || groups > OAL_MAX_GROUPS || (factor_rows != 1 && factor_rows != q_heads))
    return fail(OAL_ERR_ARGUMENT, "oal_expand_factor_grad: bad geometry");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LaunchScope scope("expand_factor_grad", st);
  cudaError_t e = oal::expand_factor_grad(factor, factor_rows, q_heads, groups, d_coef_a, d_coef_b, d_coef_c, d_factor, st);
  return e == cudaSuccess ? OAL_OK : fail_cuda(e, "oal_expand_factor_grad");
}

int oal_backward(const OalProblem* p, const void* q, const void* k, const void* v, const int32_t* dim_perm,
                 const int32_t* group_start, const float* coef_a, const float* coef_b, const float* coef_c,
                 const float* num, const float* den, const void* saved_state, const void* grad_out,
                 const float* grad_num, const float* grad_den, void* dq, void* dk, void* dv,
                 float* d_coef_a, float* d_coef_b, float* d_coef_c, const float* dstate_in, void* workspace,
                 size_t workspace_bytes, int32_t* status, void* stream) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (!q || !k || !v || !dim_perm || !group_start || !coef_a || !coef_b || !coef_c || !num || !den || !status)
    return fail(OAL_ERR_ARGUMENT, "oal_backward: NULL tensor pointer");
  const int mask = p->grad_mask;
  if ((mask & OAL_GRAD_Q) && !dq) return fail(OAL_ERR_ARGUMENT, "dq requested but NULL");
  if ((mask & OAL_GRAD_K) && !dk) return fail(OAL_ERR_ARGUMENT, "dk requested but NULL");
  if ((mask & OAL_GRAD_V) && !dv) return fail(OAL_ERR_ARGUMENT, "dv requested but NULL");
  if ((mask & OAL_GRAD_COEF) && (!d_coef_a || !d_coef_b || !d_coef_c))
    return fail(OAL_ERR_ARGUMENT, "coefficient gradients requested but NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->precision == OAL_PRECISION_FP32_IEEE) {
    if (dstate_in) return fail(OAL_ERR_ARGUMENT, "fp32_ieee mode keeps no chunk state: dstate_in must be NULL");
    BackwardSpace s = carve_backward(p, workspace);
    if (!workspace || workspace_bytes < s.bytes) return fail(OAL_ERR_WORKSPACE, "oal_backward: workspace too small");
    const size_t rows = (size_t)p->batch * p->q_heads * p->seq_len;
    cudaError_t e;
    { LaunchScope scope("norm_vjp", st);
      e = oal::norm_vjp(grad_out, p->out_dtype, grad_num, grad_den, num, den, p->floor, s.g, rows, st); }
    if (e != cudaSuccess) return fail_cuda(e, "normalisation VJP kernel");
    oal::PairArgs a = base_args(p, q, k, v, dim_perm, group_start, coef_a, coef_b, coef_c, status);
    a.g = s.g;
    if (mask & (OAL_GRAD_Q | OAL_GRAD_COEF)) {
      a.dq = (mask & OAL_GRAD_Q) ? dq : nullptr;
      a.coef_partial = (mask & OAL_GRAD_COEF) ? s.coef_pairs : nullptr;
      { LaunchScope scope("pairs_backward_q", st); e = oal::pairs_backward_q(a, st); }
      if (e != cudaSuccess) return fail_cuda(e, "backward query-side pair kernel");
      if (mask & OAL_GRAD_COEF) {
        { LaunchScope scope("reduce_coefs", st);
          e = oal::reduce_coefs(s.coef_pairs, oal::pairs_tiles(p->seq_len), nullptr, p->batch, p->q_heads,
                                p->groups, d_coef_a, d_coef_b, d_coef_c, st); }
        if (e != cudaSuccess) return fail_cuda(e, "coefficient reduction kernel");
      }
    }
    if (mask & (OAL_GRAD_K | OAL_GRAD_V)) {
      a.dq = nullptr; a.coef_partial = nullptr;
      a.dk = (mask & OAL_GRAD_K) ? dk : nullptr;
      a.dv = (mask & OAL_GRAD_V) ? dv : nullptr;
      { LaunchScope scope("pairs_backward_kv", st); e = oal::pairs_backward_kv(a, st); }
      if (e != cudaSuccess) return fail_cuda(e, "backward key/value-side pair kernel");
    }
    return OAL_OK;
  }
  // bf16_tensorcore
  if (!saved_state) return fail(OAL_ERR_ARGUMENT, "oal_backward: saved_state is NULL");
  BackwardSpaceTC s = carve_backward_tc(p, workspace);
  if (!workspace || workspace_bytes < s.bytes) return fail(OAL_ERR_WORKSPACE, "oal_backward: workspace too small");
  const int nb = chunk_count(p), units = p->batch * p->kv_heads, rep = p->q_heads / p->kv_heads;
  const bool want_q = mask & OAL_GRAD_Q, want_k = mask & OAL_GRAD_K, want_v = mask & OAL_GRAD_V;
  const bool want_c = mask & OAL_GRAD_COEF;
  const bool tc = tc_intra(p);                // intra-chunk term on the tensor cores (else token-pair kernels)
  cudaError_t e;
  if (!(mask & OAL_GRAD_REUSE_STATE_STAGE)) {
    rc = backward_state_stage(p, q, dim_perm, group_start, coef_a, coef_b, coef_c, num, den, saved_state, grad_out,
                              grad_num, grad_den, s, status, st);
    if (rc) return rc;
  }
  const void* factors = saved_factors(p, saved_state);      // written by the forward of this call
  // Three chains leave the state stage: the query side (on the caller's stream), the key/value side and
  // the reduction of the cross-chunk coefficient gradient.  They share no buffer, so the last two run on
  // the library's side streams and are joined before this function returns.
  SideStreams* side = side_streams();
  cudaStream_t skv = (want_k || want_v) ? fork_to(side, 0, st) : st;
  cudaStream_t sc = want_c ? fork_to(side, 1, st) : st;
  oal::PairArgs a = base_args(p, q, k, v, dim_perm, group_start, coef_a, coef_b, coef_c, status);
  a.window = kChunk;
  a.g = s.g;
  if (want_c) {
    { LaunchScope scope("dcoef_reduce", sc, 2);
      e = oal::dcoef_reduce(s.dcoef_partial, 2 * p->batch * nb, p->q_heads, dim_perm, group_start, s.dcoef, s.slots, sc); }
    if (e != cudaSuccess) return fail_cuda(e, "coefficient gradient reduction kernels");
    join_mark(side, 1, sc, st);
  }
  if (want_k || want_v) {
    { LaunchScope scope("state_scan_reverse", skv);
      e = oal::state_scan(s.dcarry, s.dt_img, nullptr, dstate_in, nullptr, units, nb, 1, skv); }
    if (e != cudaSuccess) return fail_cuda(e, "reverse state scan kernel");
    if (want_k) {
      { LaunchScope scope("feature_grad_k", skv);
        e = oal::feature_grad(false, k, nullptr, v, s.dt_img, nullptr, s.dk_cross, p->batch, p->kv_heads, 1,
                              p->seq_len, nb, status, skv); }
      if (e != cudaSuccess) return fail_cuda(e, "key feature gradient kernel");
    }
    if (want_v) {
      { LaunchScope scope("cross_read_k", skv);
        e = oal::cross_read(false, k, s.dt_img, nullptr, s.dv_cross, nullptr, p->batch, p->kv_heads, 1, p->seq_len,
                            nb, status, skv); }
      if (e != cudaSuccess) return fail_cuda(e, "key cross read kernel");
    }
  }
  if (want_q || want_c) {
    if (want_q) {
      { LaunchScope scope("feature_grad_q", st);
        e = oal::feature_grad(true, q, s.gimg, nullptr, saved_state, s.coef_table, s.dq_cross, p->batch, p->q_heads,
                              rep, p->seq_len, nb, status, st); }
      if (e != cudaSuccess) return fail_cuda(e, "query feature gradient kernel");
    }
    if (tc) {
      { LaunchScope scope("intra_backward_q", st);
        e = oal::intra_backward_q(q, k, v, s.gimg, factors, want_q ? dq : nullptr, want_q ? s.dq_cross : nullptr,
                                  want_c ? s.coef_pairs : nullptr, status, p->batch, p->q_heads, p->kv_heads,
                                  p->seq_len, nb, st); }
      if (e != cudaSuccess) return fail_cuda(e, "intra-chunk backward query-side kernel");
    } else {
      a.dq = want_q ? dq : nullptr;
      a.dq_init = want_q ? s.dq_cross : nullptr;
      a.coef_partial = want_c ? s.coef_pairs : nullptr;
      { LaunchScope scope("pairs_backward_q", st); e = oal::pairs_backward_q(a, st); }
      if (e != cudaSuccess) return fail_cuda(e, "backward query-side pair kernel");
    }
    if (want_c) {
      join_wait(side, 1, sc, st);
      { LaunchScope scope("reduce_coefs", st);
        const int rm = oal::intra_coef_terms();
        e = tc ? oal::intra_coef_finish(s.coef_pairs, nb, rm * (rm + 1) / 2 + rm + 1, rm, factors, s.slots, p->batch,
                                        p->q_heads, p->groups, d_coef_a, d_coef_b, d_coef_c, st)
               : oal::reduce_coefs(s.coef_pairs, oal::pairs_tiles(p->seq_len), s.slots, p->batch, p->q_heads,
                                   p->groups, d_coef_a, d_coef_b, d_coef_c, st); }
      if (e != cudaSuccess) return fail_cuda(e, "coefficient reduction kernel");
    }
  } else if (want_c) {
    join_wait(side, 1, sc, st);
  }
  if (want_k || want_v) {
    // the two intra-chunk kernels each fill the machine: the key/value one is queued after the query one
    if (tc) {
      { LaunchScope scope("intra_backward_kv", skv, 1 + (want_k ? 1 : 0) + (want_v ? 1 : 0));
        e = oal::intra_backward_kv(q, k, v, s.gimg, factors, want_k ? dk : nullptr, want_v ? dv : nullptr,
                                   want_k ? s.dk_cross : nullptr, want_v ? s.dv_cross : nullptr, s.dk_part, s.dv_part,
                                   status, p->batch, p->q_heads, p->kv_heads, p->seq_len, nb, skv); }
      if (e != cudaSuccess) return fail_cuda(e, "intra-chunk backward key/value-side kernel");
    } else {
      a.dq = nullptr; a.dq_init = nullptr; a.coef_partial = nullptr;
      a.dk = want_k ? dk : nullptr;
      a.dv = want_v ? dv : nullptr;
      a.dk_init = want_k ? s.dk_cross : nullptr;
      a.dv_init = want_v ? s.dv_cross : nullptr;
      { LaunchScope scope("pairs_backward_kv", skv); e = oal::pairs_backward_kv(a, skv); }
      if (e != cudaSuccess) return fail_cuda(e, "backward key/value-side pair kernel");
    }
    join_mark(side, 0, skv, st);
    join_wait(side, 0, skv, st);
  }
  return OAL_OK;
}

int oal_forward_local_state(const OalProblem* p, const void* k, const void* v, float* state_total, void* workspace,
                            size_t workspace_bytes, int32_t* status, void* stream) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (p->precision != OAL_PRECISION_BF16_TENSORCORE)
    return fail(OAL_ERR_DTYPE, "oal_forward_local_state: chunk states exist only in bf16_tensorcore mode");
  if (!k || !v || !state_total || !status) return fail(OAL_ERR_ARGUMENT, "oal_forward_local_state: NULL tensor pointer");
  ForwardSpaceTC s = carve_forward_tc(p, workspace);
  if (!workspace || workspace_bytes < s.bytes) return fail(OAL_ERR_WORKSPACE, "oal_forward_local_state: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int units = p->batch * p->kv_heads, nb = chunk_count(p);
  cudaError_t e;
  { LaunchScope scope("state_update", st); e = oal::state_update(k, v, s.ds, units, p->seq_len, nb, status, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state update kernel");
  { LaunchScope scope("state_total", st); e = oal::state_scan(s.ds, nullptr, nullptr, nullptr, state_total, units, nb, 0, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state total kernel");
  return OAL_OK;
}

int oal_backward_local_state(const OalProblem* p, const void* q, const int32_t* dim_perm, const int32_t* group_start,
                             const float* coef_a, const float* coef_b, const float* coef_c, const float* num,
                             const float* den, const void* saved_state, const void* grad_out, const float* grad_num,
                             const float* grad_den, float* dstate_total, void* workspace, size_t workspace_bytes,
                             int32_t* status, void* stream) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (p->precision != OAL_PRECISION_BF16_TENSORCORE)
    return fail(OAL_ERR_DTYPE, "oal_backward_local_state: chunk states exist only in bf16_tensorcore mode");
  if (!q || !dim_perm || !group_start || !coef_a || !coef_b || !coef_c || !num || !den || !saved_state || !dstate_total || !status)
    return fail(OAL_ERR_ARGUMENT, "oal_backward_local_state: NULL tensor pointer");
  BackwardSpaceTC s = carve_backward_tc(p, workspace);
  if (!workspace || workspace_bytes < s.bytes) return fail(OAL_ERR_WORKSPACE, "oal_backward_local_state: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OalProblem local = *p;
  local.grad_mask |= OAL_GRAD_K;      // dCarry is needed whatever the caller finally asks for
  rc = backward_state_stage(&local, q, dim_perm, group_start, coef_a, coef_b, coef_c, num, den, saved_state, grad_out,
                            grad_num, grad_den, s, status, st);
  if (rc) return rc;
  cudaError_t e;
  { LaunchScope scope("state_total", st);
    e = oal::state_scan(s.dcarry, nullptr, nullptr, nullptr, dstate_total, p->batch * p->kv_heads, chunk_count(p), 1, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state gradient total kernel");
  return OAL_OK;
}

// ---------------------------------------------------------------------------------------------
// Forward with library-owned scratch (no caller workspace, no allocation of any kind).
//
// Some hosts of this library cannot obtain device memory at call time: an inference server whose
// memory pool was carved up and frozen at start-up, a plugin that runs inside someone else's
// allocator-free execution callback, a process near its memory limit where cudaMalloc may fail or
// stall.  For them the tensor-core forward keeps its two scratch buffers -- the per-head coefficient
// table and the per-chunk state increments -- in the file-scope device array below.  The array has
// a fixed size, so the entry point only accepts problems up to kStaticMaxUnitChunks (batch x KV heads
// x 128-token chunks) and kStaticMaxHeads query heads; every GPU that loads the library holds the
// array (about 13.1 MB) until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr int kStaticMaxUnitChunks = 16;
constexpr int kStaticMaxHeads = 64;
constexpr size_t kStaticStateFloats = (size_t)kStaticMaxUnitChunks * OAL_STATE_ROWS * OAL_E_PAD;
constexpr size_t kStaticTableFloats = (size_t)kStaticMaxHeads * OAL_STATE_ROWS;
static __device__ __align__(256) float g_static_scratch[kStaticTableFloats + kStaticStateFloats];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device, resolved once per device.  In host code
// the array's name is only a handle for the runtime, not an address a kernel could use.
int static_scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(OAL_ERR_ARGUMENT, "device ordinal out of range for the static scratch table");
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return OAL_OK;
}
}  // namespace

int oal_forward_static_scratch(const OalProblem* p, const void* q, const void* k, const void* v,
                               const int32_t* dim_perm, const int32_t* group_start, const float* coef_a,
                               const float* coef_b, const float* coef_c, void* out, float* num, float* den,
                               void* saved_state, int32_t* status, void* stream) {
  int rc = check_problem(p);
  if (rc) return rc;
  if (p->precision != OAL_PRECISION_BF16_TENSORCORE)
    return fail(OAL_ERR_DTYPE, "oal_forward_static_scratch: only bf16_tensorcore uses scratch memory (fp32_ieee forward needs none: call oal_forward)");
  if (!q || !k || !v || !dim_perm || !group_start || !coef_a || !coef_b || !coef_c || !out || !num || !den || !status || !saved_state)
    return fail(OAL_ERR_ARGUMENT, "oal_forward_static_scratch: NULL tensor pointer");
  const int units = p->batch * p->kv_heads, nb = chunk_count(p);
  if ((long long)units * nb > kStaticMaxUnitChunks)
    return fail(OAL_ERR_WORKSPACE, "oal_forward_static_scratch: batch x kv_heads x ceil(seq_len/128) exceeds the static scratch limit of 16; use oal_forward with a caller workspace");
  if (p->q_heads > kStaticMaxHeads)
    return fail(OAL_ERR_WORKSPACE, "oal_forward_static_scratch: more than 64 query heads; use oal_forward with a caller workspace");
  float* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  float* coef_table = scratch;
  float* ds = scratch + kStaticTableFloats;
  void* factors = saved_factors(p, saved_state);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  { LaunchScope scope("coef_table", st, 1, false);
    e = oal::build_coef_table(dim_perm, group_start, coef_a, coef_b, coef_c, p->q_heads, p->groups, p->scale, coef_table, st); }
  if (e != cudaSuccess) return fail_cuda(e, "coefficient table kernel");
  { LaunchScope scope("state_update", st, 1, false); e = oal::state_update(k, v, ds, units, p->seq_len, nb, status, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state update kernel");
  { LaunchScope scope("state_scan", st, 1, false); e = oal::state_scan(ds, saved_state, saved_remainders(p, saved_state), nullptr, nullptr, units, nb, 0, st); }
  if (e != cudaSuccess) return fail_cuda(e, "state scan kernel");
  { LaunchScope scope("cross_read_q", st, 1, false);
    e = oal::cross_read(true, q, saved_state, coef_table, num, den, p->batch, p->q_heads, p->q_heads / p->kv_heads,
                        p->seq_len, nb, status, st); }
  if (e != cudaSuccess) return fail_cuda(e, "cross read kernel");
  if (tc_intra(p)) {
    if (int rc2 = make_head_factors(p, dim_perm, group_start, coef_a, coef_b, coef_c, factors, st, false)) return rc2;
    { LaunchScope scope("intra_forward", st, 1, false);
      e = oal::intra_forward(q, k, v, factors, out, num, den, status, p->batch, p->q_heads, p->kv_heads, p->seq_len, nb,
                             p->out_dtype, p->floor, (p->flags & OAL_FLAG_OUT_TOKEN_MAJOR) != 0, st); }
    if (e != cudaSuccess) return fail_cuda(e, "intra-chunk forward kernel");
    return OAL_OK;
  }
  oal::PairArgs a = base_args(p, q, k, v, dim_perm, group_start, coef_a, coef_b, coef_c, status);
  a.window = kChunk;
  a.out = out; a.num = num; a.den = den; a.accumulate = 1;
  { LaunchScope scope("pairs_forward", st, 1, false); e = oal::pairs_forward(a, st); }
  if (e != cudaSuccess) return fail_cuda(e, "forward pair kernel");
  return OAL_OK;
}

}  // extern "C"
