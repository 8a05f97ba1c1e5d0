// chill_fwd_bwd_host: forward + backward for tensors that live in host memory.
//
// The batch is cut into chunks of whole kv-head groups of one batch row; a chunk is uploaded on one stream,
// computed on a second (chill_fwd, chill_bwd_delta, chill_bwd of this library) and downloaded on a third, over
// two sets of device staging buffers, so the PCIe transfers of both directions overlap each other and the
// kernels.  Only the public entry points of the library and the CUDA runtime are used here.
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

#include "../../include/chill_b200.h"

namespace chill {
int record_cuda_failure(cudaError_t e, const char* what);  // chill_abi.cu: fills chill_last_cuda_error()

namespace {

constexpr int kSlots = 2;
constexpr size_t kAlign = 256;
constexpr double kDefaultChunkBytes = 40e6;

struct Pipeline {
  cudaStream_t in = nullptr, cmp = nullptr, out = nullptr;
  cudaEvent_t start = nullptr, done[3] = {nullptr, nullptr, nullptr};
  // per slot: inputs uploaded, backward finished, downloads finished
  cudaEvent_t up[kSlots], bwd[kSlots], down[kSlots];
  bool ready = false;
  std::mutex mu;  // one call at a time per device builds its schedule on these streams
};

Pipeline* pipeline_of_current_device() {
  constexpr int kMaxDevices = 64;
  static Pipeline cache[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  Pipeline& p = cache[dev];
  if (!p.ready) {
    bool ok = cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.cmp, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking) == cudaSuccess;
    auto ev = [&](cudaEvent_t* e) { ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess; };
    ev(&p.start);
    for (auto& e : p.done) ev(&e);
    for (int s = 0; s < kSlots; ++s) {
      ev(&p.up[s]);
      ev(&p.bwd[s]);
      ev(&p.down[s]);
    }
    if (!ok) return nullptr;
    p.ready = true;
  }
  return &p;
}

size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }
size_t esize(int dtype) { return dtype == CHILL_F32 ? 4 : 2; }

// kv-head groups per full-size chunk
int groups_per_chunk(const chill_host_args& a) {
  const chill_shape& s = a.s;
  if (a.chunk_groups > 0) return a.chunk_groups < s.H_kv ? a.chunk_groups : s.H_kv;
  const int G = s.H / s.H_kv;
  const double per_group = (double)s.Lq * s.D * esize(s.dtype) * (2.0 * G + 2.0);  // q, d_o: G heads; k, v: one
  int big = (int)(kDefaultChunkBytes / per_group);
  if (big < 1) big = 1;
  if (big > s.H_kv) big = s.H_kv;
  // even split of a batch row into the same number of chunks
  const int n_chunks = (s.H_kv + big - 1) / big;
  return (s.H_kv + n_chunks - 1) / n_chunks;
}

struct Chunk {
  int b, g0, n;
};

// Every (batch row, kv-head group) once, in order: each batch row in chunks of `big` groups.
// (Schedules that start and end with smaller chunks, to shorten the first upload and the last download that
// nothing overlaps, were measured and lost: a small chunk costs as much kernel time as a large one, ~0.2 ms.)
std::vector<Chunk> schedule(int B, int groups, int big) {
  std::vector<Chunk> out;
  for (int b = 0; b < B; ++b)
    for (int g0 = 0; g0 < groups; g0 += big) out.push_back({b, g0, groups - g0 < big ? groups - g0 : big});
  return out;
}

// Staging buffers of one slot, sized for the largest chunk.
struct SlotLayout {
  size_t q, k, v, d_o, o, dq, dk, dv, lse, delta, accum, total;
};

chill_shape chunk_shape(const chill_shape& s, int groups) {
  chill_shape c = s;
  c.B = 1;
  c.H_kv = groups;
  c.H = groups * (s.H / s.H_kv);
  c.flags = s.flags & ~CHILL_FLAG_BWD_DETERMINISTIC;
  return c;
}

SlotLayout slot_layout(const chill_shape& s, int big) {
  const int G = s.H / s.H_kv;
  const size_t head = (size_t)s.Lq * s.D * esize(s.dtype);
  const size_t qb = round_up(head * G * big), kb = round_up(head * big);
  const size_t rows = round_up((size_t)G * big * s.Lq * sizeof(float));
  SlotLayout l;
  size_t off = 0;
  auto take = [&](size_t n) {
    const size_t at = off;
    off += n;
    return at;
  };
  l.q = take(qb);
  l.k = take(kb);
  l.v = take(kb);
  l.d_o = take(qb);
  l.o = take(qb);
  l.dq = take(qb);
  l.dk = take(kb);
  l.dv = take(kb);
  l.lse = take(rows);
  l.delta = take(rows);
  const chill_shape c = chunk_shape(s, big);
  l.accum = take((s.flags & CHILL_FLAG_BWD_DETERMINISTIC) ? 0 : round_up(chill_bwd_dq_accum_bytes(&c)));
  l.total = off;
  return l;
}

int check(const chill_host_args* a) {
  if (a == nullptr) return CHILL_E_INVALID;
  const chill_shape& s = a->s;
  if (s.B <= 0 || s.H <= 0 || s.H_kv <= 0 || s.H % s.H_kv != 0 || s.Lq <= 0 || s.D <= 0) return CHILL_E_INVALID;
  if (s.Lq != s.Lk || s.seq_len != s.Lq || s.q_offset != 0 || s.k_offset != 0 || s.lens != nullptr) return CHILL_E_INVALID;
  if (s.dtype != CHILL_F32 && s.dtype != CHILL_F16 && s.dtype != CHILL_BF16) return CHILL_E_INVALID;
  return CHILL_OK;
}

void contiguous_strides(int64_t* st, int H, int L, int D) {
  st[0] = (int64_t)H * L * D;
  st[1] = (int64_t)L * D;
  st[2] = D;
  st[3] = 1;
}

}  // namespace
}  // namespace chill

extern "C" size_t chill_host_workspace_bytes(const chill_host_args* a) {
  using namespace chill;
  if (check(a) != CHILL_OK) return 0;
  return kSlots * slot_layout(a->s, groups_per_chunk(*a)).total;
}

extern "C" int chill_host_chunk_schedule(const chill_host_args* a, int32_t* out, int32_t capacity) {
  using namespace chill;
  const int rc = check(a);
  if (rc != CHILL_OK) return rc;
  const std::vector<Chunk> chunks = schedule(a->s.B, a->s.H_kv, groups_per_chunk(*a));
  for (size_t i = 0; i < chunks.size() && out != nullptr && (int32_t)i < capacity; ++i) {
    out[3 * i] = chunks[i].b;
    out[3 * i + 1] = chunks[i].g0;
    out[3 * i + 2] = chunks[i].n;
  }
  return (int)chunks.size();
}

extern "C" int chill_fwd_bwd_host(const chill_host_args* a, void* stream) {
  using namespace chill;
  int rc = check(a);
  if (rc != CHILL_OK) return rc;
  const chill_shape& s = a->s;
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->d_o == nullptr || a->o == nullptr ||
      a->dq == nullptr || a->dk == nullptr || a->dv == nullptr || a->workspace == nullptr)
    return CHILL_E_INVALID;
  const int big = groups_per_chunk(*a);
  const SlotLayout lay = slot_layout(s, big);
  if (a->workspace_bytes < kSlots * lay.total || ((uintptr_t)a->workspace & (kAlign - 1)) != 0) return CHILL_E_INVALID;
  Pipeline* p = pipeline_of_current_device();
  if (p == nullptr) return record_cuda_failure(cudaGetLastError(), "host pipeline streams");
  std::lock_guard<std::mutex> lock(p->mu);
  cudaStream_t user = static_cast<cudaStream_t>(stream);
  const int G = s.H / s.H_kv;
  const size_t head = (size_t)s.Lq * s.D * esize(s.dtype);
  const bool deterministic = (s.flags & CHILL_FLAG_BWD_DETERMINISTIC) != 0;

#define CHILL_CUDA(call, what)                              \
  do {                                                      \
    cudaError_t e_ = (call);                                \
    if (e_ != cudaSuccess) return record_cuda_failure(e_, what); \
  } while (0)

  CHILL_CUDA(cudaEventRecord(p->start, user), "event record");
  CHILL_CUDA(cudaStreamWaitEvent(p->in, p->start, 0), "stream wait");
  CHILL_CUDA(cudaStreamWaitEvent(p->cmp, p->start, 0), "stream wait");
  CHILL_CUDA(cudaStreamWaitEvent(p->out, p->start, 0), "stream wait");

  const std::vector<Chunk> chunks = schedule(s.B, s.H_kv, big);
  for (size_t i = 0; i < chunks.size(); ++i) {
    const Chunk& c = chunks[i];
    const int slot = (int)(i % kSlots);
    const bool reused = i >= (size_t)kSlots;
    char* base = static_cast<char*>(a->workspace) + slot * lay.total;
    const int nh = c.n * G;
    const size_t q_off = ((size_t)c.b * s.H + (size_t)c.g0 * G) * head, q_bytes = (size_t)nh * head;
    const size_t k_off = ((size_t)c.b * s.H_kv + c.g0) * head, k_bytes = (size_t)c.n * head;

    // ---- upload
    if (reused) CHILL_CUDA(cudaStreamWaitEvent(p->in, p->bwd[slot], 0), "stream wait");  // inputs consumed
    CHILL_CUDA(cudaMemcpyAsync(base + lay.q, (const char*)a->q + q_off, q_bytes, cudaMemcpyHostToDevice, p->in), "upload q");
    CHILL_CUDA(cudaMemcpyAsync(base + lay.k, (const char*)a->k + k_off, k_bytes, cudaMemcpyHostToDevice, p->in), "upload k");
    CHILL_CUDA(cudaMemcpyAsync(base + lay.v, (const char*)a->v + k_off, k_bytes, cudaMemcpyHostToDevice, p->in), "upload v");
    CHILL_CUDA(cudaMemcpyAsync(base + lay.d_o, (const char*)a->d_o + q_off, q_bytes, cudaMemcpyHostToDevice, p->in), "upload dO");
    CHILL_CUDA(cudaEventRecord(p->up[slot], p->in), "event record");

    // ---- kernels
    chill_bwd_args bw = {};
    bw.s = chunk_shape(s, c.n);
    bw.q = base + lay.q;
    bw.k = base + lay.k;
    bw.v = base + lay.v;
    bw.o = base + lay.o;
    bw.d_o = base + lay.d_o;
    bw.lse = reinterpret_cast<float*>(base + lay.lse);
    bw.delta = reinterpret_cast<float*>(base + lay.delta);
    bw.dq = base + lay.dq;
    bw.dk = base + lay.dk;
    bw.dv = base + lay.dv;
    bw.dq_accum = deterministic ? nullptr : reinterpret_cast<float*>(base + lay.accum);
    if (!deterministic && chill_bwd_dq_accum_bytes(&bw.s) == 0) bw.dq_accum = nullptr;
    for (int64_t* st : {bw.q_strides, bw.o_strides, bw.do_strides, bw.dq_strides}) contiguous_strides(st, nh, s.Lq, s.D);
    for (int64_t* st : {bw.k_strides, bw.v_strides, bw.dk_strides, bw.dv_strides}) contiguous_strides(st, c.n, s.Lq, s.D);
    bw.lse_strides[0] = (int64_t)nh * s.Lq;
    bw.lse_strides[1] = s.Lq;
    bw.lse_strides[2] = 1;
    chill_fwd_args fw = {};
    fw.s = bw.s;
    fw.q = bw.q;
    fw.k = bw.k;
    fw.v = bw.v;
    fw.o = base + lay.o;
    fw.lse = reinterpret_cast<float*>(base + lay.lse);
    for (int j = 0; j < 4; ++j) {
      fw.q_strides[j] = bw.q_strides[j];
      fw.k_strides[j] = bw.k_strides[j];
      fw.v_strides[j] = bw.v_strides[j];
      fw.o_strides[j] = bw.o_strides[j];
    }
    for (int j = 0; j < 3; ++j) fw.lse_strides[j] = bw.lse_strides[j];

    CHILL_CUDA(cudaStreamWaitEvent(p->cmp, p->up[slot], 0), "stream wait");
    if (reused) CHILL_CUDA(cudaStreamWaitEvent(p->cmp, p->down[slot], 0), "stream wait");  // outputs downloaded
    if ((rc = chill_fwd(&fw, p->cmp)) != CHILL_OK) return rc;
    if ((rc = chill_bwd_delta(&bw, p->cmp)) != CHILL_OK) return rc;
    if ((rc = chill_bwd(&bw, p->cmp)) != CHILL_OK) return rc;
    CHILL_CUDA(cudaEventRecord(p->bwd[slot], p->cmp), "event record");

    // ---- download
    // (Starting the forward before dO has arrived, or sending O back while the backward runs, measured 15 % slower
    // end to end: the uploads slow down when more of the kernel time overlaps them.)
    CHILL_CUDA(cudaStreamWaitEvent(p->out, p->bwd[slot], 0), "stream wait");
    CHILL_CUDA(cudaMemcpyAsync((char*)a->o + q_off, base + lay.o, q_bytes, cudaMemcpyDeviceToHost, p->out), "download o");
    CHILL_CUDA(cudaMemcpyAsync((char*)a->dq + q_off, base + lay.dq, q_bytes, cudaMemcpyDeviceToHost, p->out), "download dq");
    CHILL_CUDA(cudaMemcpyAsync((char*)a->dk + k_off, base + lay.dk, k_bytes, cudaMemcpyDeviceToHost, p->out), "download dk");
    CHILL_CUDA(cudaMemcpyAsync((char*)a->dv + k_off, base + lay.dv, k_bytes, cudaMemcpyDeviceToHost, p->out), "download dv");
    CHILL_CUDA(cudaEventRecord(p->down[slot], p->out), "event record");
  }

  cudaStream_t all[3] = {p->in, p->cmp, p->out};
  for (int j = 0; j < 3; ++j) {
    CHILL_CUDA(cudaEventRecord(p->done[j], all[j]), "event record");
    CHILL_CUDA(cudaStreamWaitEvent(user, p->done[j], 0), "stream wait");
  }
#undef CHILL_CUDA
  return CHILL_OK;
}
