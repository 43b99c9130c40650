// Multi-GPU shim of the matmul path on one box.
//
// The reference has no multi-device operator: its model is one Device per GPU, each driven by
// its own thread and session (tfcc/core/utils/tfcc_initializer.cpp:50-66,
// tfcc/cuda/utils/tfcc_cudautils.cpp:23-50).  What is added here is the N split of one large
// product: GPU g holds A and the column shard B[:, g*N/G:(g+1)*N/G], multiplies it on the
// tensor-core path and stores every finished tile into the same columns of EVERY GPU's
// row-major C with ordinary stores over NVLink (tfccb200_*_nsplit_push), so that each GPU ends
// up with the whole C and no separate all-gather runs.
//
// Two ways to drive it:
//   * one process per GPU (torch.distributed, MPI, ...): the caller maps its peers' buffers
//     (CUDA IPC, symmetric memory) and calls the per-rank entry points, passing a barrier
//     callback where a cross-rank barrier is needed (tfccb200_sgemm_nsplit_host);
//   * one process for all GPUs -- how a TFCC program with one Device per GPU looks: a
//     tfccb200_group enables peer access between its devices, owns one stream per device and
//     orders the devices with events (tfccb200_group_*).
// Nothing here uses a TMA or multicast LOAD on peer memory; peers are only ever written, with
// st.global or multimem.st.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <new>
#include <vector>

#include "internal.h"
#include "pdl.cuh"

namespace tfccb200 {

namespace {

// dst[d][i] = src[i] for every destination: one pass over the source, 128 bits per thread.
// With `mc` set the line is stored once through the NVLink multicast alias instead.
struct BroadcastTargets {
  float4* dst[8];
  unsigned num_dst;
  float4* mc;
};

__global__ void __launch_bounds__(256)
broadcast_kernel(const float4* __restrict__ src, BroadcastTargets t, size_t n4) {
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n4; i += gridDim.x * 256ull) {
    const float4 v = __ldcs(src + i);
    if (t.mc) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                   :
                   : "l"(t.mc + i), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                   : "memory");
    } else {
      for (unsigned d = 0; d < t.num_dst; ++d) t.dst[d][i] = v;
    }
  }
}

int broadcast_bytes(cudaStream_t stream, const void* src, void* const* dst, unsigned num_dst,
                    void* mc, size_t bytes) {
  if (bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15u)) return TFCCB200_EALIGN;
  BroadcastTargets t = {};
  for (unsigned d = 0; d < num_dst; ++d) {
    if (reinterpret_cast<uintptr_t>(dst[d]) & 15u) return TFCCB200_EALIGN;
    t.dst[t.num_dst++] = static_cast<float4*>(dst[d]);
  }
  t.mc = static_cast<float4*>(mc);
  if (t.num_dst == 0 && !t.mc) return TFCCB200_OK;
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const size_t n4 = bytes / 16;
  size_t blocks = (n4 + 255) / 256;
  blocks = std::min<size_t>(blocks, static_cast<size_t>(di->sm_count) * 8);
  broadcast_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const float4*>(src), t, n4);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

}  // namespace

// ---- one rank's share of an N-split product whose operands start in host memory ----------
//
// The rank's M/G rows are cut into `blocks` row blocks of Rb rows.  Step p multiplies row block p
// of EVERY rank, so the staging buffers are laid out step by step: block p of rank q lives at
// staging rows [p*G*Rb + q*Rb, +Rb) of A and of C, which makes the operand of step p one
// contiguous [G*Rb, K] matrix and this rank's result rows of step p one contiguous piece.  Four
// streams per rank:
//   up:    A block 0, the B shard, A blocks 1.. from host memory
//   xch:   block p stored on into every peer's staging once it has arrived
//   main:  barrier, product of step p (tiles pushed into every rank's C staging), barrier, ...
//   down:  this rank's rows of step p to host memory once the barrier after the product says
//          that every rank's tiles have landed
// so that the uploads of later blocks and the downloads of earlier ones run under the products.
cudaError_t HostLanes::create() {
  cudaError_t e;
  for (cudaStream_t* s : {&up, &xch, &down})
    if ((e = cudaStreamCreateWithFlags(s, cudaStreamNonBlocking)) != cudaSuccess) return e;
  for (cudaEvent_t* ev : {&start, &b_up, &tail})
    if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return e;
  for (unsigned p = 0; p < kMaxHostBlocks; ++p)
    for (cudaEvent_t* ev : {&a_up[p], &a_sent[p], &c_whole[p]})
      if ((e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming)) != cudaSuccess) return e;
  return cudaSuccess;
}

void HostLanes::join() {
  for (cudaStream_t s : {up, xch, down})
    if (s) cudaStreamSynchronize(s);
}

void HostLanes::destroy() {
  join();
  for (cudaEvent_t* ev : {&start, &b_up, &tail})
    if (*ev) cudaEventDestroy(*ev), *ev = nullptr;
  for (unsigned p = 0; p < kMaxHostBlocks; ++p)
    for (cudaEvent_t* ev : {&a_up[p], &a_sent[p], &c_whole[p]})
      if (*ev) cudaEventDestroy(*ev), *ev = nullptr;
  for (cudaStream_t* s : {&up, &xch, &down})
    if (*s) cudaStreamDestroy(*s), *s = nullptr;
}

namespace {

#define HOST_TRY(expr)                                        \
  do {                                                        \
    cudaError_t e_ = (expr);                                  \
    if (e_ != cudaSuccess) return static_cast<int>(e_);       \
  } while (0)

struct HostBlocks {
  unsigned G, rows, rb, step_rows;
  size_t n_total;
};

HostBlocks host_blocks(const NsplitHostRank& r, unsigned blocks) {
  HostBlocks h;
  h.G = r.num_ranks;
  h.rows = r.M / r.num_ranks;
  h.rb = h.rows / blocks;
  h.step_rows = h.rb * h.G;
  h.n_total = static_cast<size_t>(r.N_shard) * r.num_ranks;
  return h;
}

int host_download(const NsplitHostRank& r, const HostBlocks& h, unsigned p) {
  HostLanes& L = *r.lanes;
  HOST_TRY(cudaEventRecord(L.c_whole[p], r.stream));
  HOST_TRY(cudaStreamWaitEvent(L.down, L.c_whole[p], 0));
  const float* src = r.C_ranks[r.rank] +
                     (static_cast<size_t>(p) * h.step_rows + static_cast<size_t>(r.rank) * h.rb) * h.n_total;
  HOST_TRY(cudaMemcpyAsync(r.hC_rows + static_cast<size_t>(p) * h.rb * h.n_total, src,
                           static_cast<size_t>(h.rb) * h.n_total * 4, cudaMemcpyDeviceToHost, L.down));
  return TFCCB200_OK;
}

}  // namespace

// Row blocks of about 256 rows per rank: the call is bound by the host side of the transfers,
// so finer blocks (more of the uploads and downloads under one another) beat fuller products
// (measured for 8192^3, blocks of 512 / 256 / 128 rows: 5.80 / 5.44 / 5.33 ms on eight GPUs,
// 5.05 / 5.09 / 5.17 on four, 8.35 / 8.12 / 7.96 on two).  At most kMaxHostBlocks, and a count
// that divides the rank's rows.
unsigned nsplit_host_blocks(const NsplitHostRank& r) {
  const unsigned rows = r.M / r.num_ranks;
  unsigned want = std::min(kMaxHostBlocks, std::max(1u, rows / 256));
  if (const char* env = std::getenv("TFCCB200_HOST_BLOCKS")) {
    const int v = std::atoi(env);
    if (v >= 1) want = std::min<unsigned>(kMaxHostBlocks, static_cast<unsigned>(v));
  }
  while (want > 1 && rows % want != 0) --want;
  return want;
}

int nsplit_host_start(const NsplitHostRank& r, unsigned blocks) {
  const HostBlocks h = host_blocks(r, blocks);
  HostLanes& L = *r.lanes;
  // the side streams begin behind whatever the caller queued on the product stream
  HOST_TRY(cudaEventRecord(L.start, r.stream));
  for (cudaStream_t s : {L.up, L.xch, L.down}) HOST_TRY(cudaStreamWaitEvent(s, L.start, 0));
  const size_t block_elems = static_cast<size_t>(h.rb) * r.K;
  for (unsigned p = 0; p < blocks; ++p) {
    const size_t at = (static_cast<size_t>(p) * h.step_rows + static_cast<size_t>(r.rank) * h.rb) * r.K;
    float* mine = r.A_ranks[r.rank] + at;
    HOST_TRY(cudaMemcpyAsync(mine, r.hA_rows + static_cast<size_t>(p) * block_elems, block_elems * 4,
                             cudaMemcpyHostToDevice, L.up));
    HOST_TRY(cudaEventRecord(L.a_up[p], L.up));
    if (p == 0) {  // B behind the first block: the first exchange runs while it crosses PCIe
      HOST_TRY(cudaMemcpy2DAsync(r.B_shard_dev, static_cast<size_t>(r.N_shard) * 4, r.hB_shard,
                                 static_cast<size_t>(r.ldb_host) * 4,
                                 static_cast<size_t>(r.N_shard) * 4, r.K, cudaMemcpyHostToDevice,
                                 L.up));
      HOST_TRY(cudaEventRecord(L.b_up, L.up));
    }
    HOST_TRY(cudaStreamWaitEvent(L.xch, L.a_up[p], 0));
    void* dst[8];
    unsigned n = 0;
    for (unsigned d = 0; d < r.num_ranks; ++d)
      if (d != r.rank && r.A_ranks[d]) dst[n++] = r.A_ranks[d] + at;
    void* mc = r.A_multicast ? r.A_multicast + at : nullptr;
    int st = broadcast_bytes(L.xch, mine, dst, n, mc, block_elems * 4);
    if (st != TFCCB200_OK) return st;
    HOST_TRY(cudaEventRecord(L.a_sent[p], L.xch));
  }
  return TFCCB200_OK;
}

// Before barrier p (p < blocks): this rank's block p must have reached every peer.
int nsplit_host_before_barrier(const NsplitHostRank& r, unsigned blocks, unsigned p) {
  if (p >= blocks) return TFCCB200_OK;
  HOST_TRY(cudaStreamWaitEvent(r.stream, r.lanes->a_sent[p], 0));
  return TFCCB200_OK;
}

// Behind barrier p: every rank's tiles of step p-1 have landed (download them) and every
// rank's A block p has arrived (multiply it).  Barrier 0 also says that the peers have finished
// reading the C staging of their previous call.  p == blocks closes the call.
int nsplit_host_after_barrier(const NsplitHostRank& r, unsigned blocks, unsigned p) {
  const HostBlocks h = host_blocks(r, blocks);
  HostLanes& L = *r.lanes;
  if (p > 0) {
    int st = host_download(r, h, p - 1);
    if (st != TFCCB200_OK) return st;
  }
  if (p == blocks) {
    HOST_TRY(cudaEventRecord(L.tail, L.down));
    HOST_TRY(cudaStreamWaitEvent(r.stream, L.tail, 0));
    return TFCCB200_OK;
  }
  if (p == 0) HOST_TRY(cudaStreamWaitEvent(r.stream, L.b_up, 0));
  const size_t a_at = static_cast<size_t>(p) * h.step_rows * r.K;
  const size_t c_at = static_cast<size_t>(p) * h.step_rows * h.n_total;
  float* c_step[8];
  for (unsigned d = 0; d < r.num_ranks; ++d) c_step[d] = r.C_ranks[d] ? r.C_ranks[d] + c_at : nullptr;
  return tfccb200_sgemm_nsplit_push(r.stream, r.A_ranks[r.rank] + a_at, r.B_shard_dev, c_step,
                                    r.num_ranks, r.rank, nullptr, h.step_rows, r.N_shard, r.K,
                                    r.precision, r.C_multicast ? r.C_multicast + c_at : nullptr,
                                    r.workspace, r.workspace_bytes, r.status);
}

int nsplit_host_check(const NsplitHostRank& r) {
  if (!r.hA_rows || !r.hB_shard || !r.hC_rows || !r.A_ranks || !r.B_shard_dev || !r.C_ranks)
    return TFCCB200_EINVAL;
  if (r.num_ranks == 0 || r.num_ranks > 8 || r.rank >= r.num_ranks) return TFCCB200_EINVAL;
  if (r.M == 0 || r.N_shard == 0 || r.K == 0 || r.M % r.num_ranks != 0) return TFCCB200_EINVAL;
  if (r.ldb_host < r.N_shard) return TFCCB200_EINVAL;
  if (r.K % 4 != 0 || r.N_shard % 4 != 0) return TFCCB200_EALIGN;
  if (!r.A_ranks[r.rank] || !r.C_ranks[r.rank]) return TFCCB200_EINVAL;
  return TFCCB200_OK;
}

}  // namespace tfccb200

using namespace tfccb200;

// ---- the in-process device group -------------------------------------------------------------
struct tfccb200_group {
  int ndev = 0;
  int dev[8] = {};
  cudaStream_t stream[8] = {};
  cudaEvent_t done[8] = {};      // "everything queued on stream[i] so far"
  HostLanes lanes[8];            // side streams of the host-buffer path
  int* status[8] = {};           // device status words
  void* workspace[8] = {};
  size_t workspace_bytes[8] = {};
  // staging of the host-buffer entry point, grown on demand and kept
  float* A[8] = {};
  float* B[8] = {};
  float* C[8] = {};
  size_t a_elems = 0, b_elems = 0, c_elems = 0;
};

namespace {

struct DeviceScope {  // restores the caller's current device
  int saved = -1;
  DeviceScope() { cudaGetDevice(&saved); }
  ~DeviceScope() {
    if (saved >= 0) cudaSetDevice(saved);
  }
};

// Every stream of the group waits for everything queued so far on all the others.
cudaError_t group_barrier(tfccb200_group* g) {
  cudaError_t e;
  for (int i = 0; i < g->ndev; ++i) {
    if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return e;
    if ((e = cudaEventRecord(g->done[i], g->stream[i])) != cudaSuccess) return e;
  }
  for (int j = 0; j < g->ndev; ++j) {
    if ((e = cudaSetDevice(g->dev[j])) != cudaSuccess) return e;
    for (int i = 0; i < g->ndev; ++i)
      if (i != j && (e = cudaStreamWaitEvent(g->stream[j], g->done[i], 0)) != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t grow(float** p, size_t elems) {
  if (*p) cudaFree(*p);
  *p = nullptr;
  return cudaMalloc(reinterpret_cast<void**>(p), elems * sizeof(float));
}

// Status of the device status words (and of the streams): TFCCB200_EDEVICE if a kernel of the
// group abandoned a wait.  Synchronises every stream.
int group_finish(tfccb200_group* g) {
  int result = TFCCB200_OK;
  for (int i = 0; i < g->ndev; ++i) {
    cudaError_t e;
    if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return static_cast<int>(e);
    int word = 0;
    if ((e = cudaMemcpyAsync(&word, g->status[i], sizeof(int), cudaMemcpyDeviceToHost,
                             g->stream[i])) != cudaSuccess)
      return static_cast<int>(e);
    if ((e = cudaStreamSynchronize(g->stream[i])) != cudaSuccess) return static_cast<int>(e);
    if (word) {
      cudaMemsetAsync(g->status[i], 0, sizeof(int), g->stream[i]);
      result = TFCCB200_EDEVICE;
    }
  }
  return result;
}

// The calling thread's side streams on the current device, made on first use and kept until
// the thread ends (a per-call set would cost more than a small product).
constexpr int kLaneDevices = 16;
HostLanes* thread_lanes(cudaError_t* err) {
  struct PerThread {
    HostLanes lanes[kLaneDevices];
    bool made[kLaneDevices] = {};
    ~PerThread() {
      int saved = -1;
      if (cudaGetDevice(&saved) != cudaSuccess) return;  // the runtime is already gone
      for (int d = 0; d < kLaneDevices; ++d)
        if (made[d] && cudaSetDevice(d) == cudaSuccess) lanes[d].destroy();
      cudaSetDevice(saved);
    }
  };
  static thread_local PerThread t;
  int dev = -1;
  if ((*err = cudaGetDevice(&dev)) != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kLaneDevices) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  if (!t.made[dev]) {
    if ((*err = t.lanes[dev].create()) != cudaSuccess) {
      t.lanes[dev].destroy();
      return nullptr;
    }
    t.made[dev] = true;
  }
  return &t.lanes[dev];
}

}  // namespace

extern "C" {

int tfccb200_group_create(int ndev, const int* devices, tfccb200_group** out) {
  if (!devices || !out || ndev < 1 || ndev > 8) return TFCCB200_EINVAL;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return static_cast<int>(e);
  for (int i = 0; i < ndev; ++i)
    if (devices[i] < 0 || devices[i] >= count) return TFCCB200_EINVAL;
  DeviceScope scope;
  tfccb200_group* g = new (std::nothrow) tfccb200_group;
  if (!g) return static_cast<int>(cudaErrorMemoryAllocation);
  g->ndev = ndev;
  for (int i = 0; i < ndev; ++i) g->dev[i] = devices[i];
  auto fail = [&](int st) {
    tfccb200_group_destroy(g);
    return st;
  };
  for (int i = 0; i < ndev; ++i) {
    if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return fail(static_cast<int>(e));
    for (int j = 0; j < ndev; ++j) {
      if (g->dev[j] == g->dev[i]) continue;
      int can = 0;
      if ((e = cudaDeviceCanAccessPeer(&can, g->dev[i], g->dev[j])) != cudaSuccess)
        return fail(static_cast<int>(e));
      if (!can) return fail(TFCCB200_EUNSUPPORTED);
      e = cudaDeviceEnablePeerAccess(g->dev[j], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
      } else if (e != cudaSuccess) {
        return fail(static_cast<int>(e));
      }
    }
    if ((e = cudaStreamCreateWithFlags(&g->stream[i], cudaStreamNonBlocking)) != cudaSuccess)
      return fail(static_cast<int>(e));
    if ((e = cudaEventCreateWithFlags(&g->done[i], cudaEventDisableTiming)) != cudaSuccess)
      return fail(static_cast<int>(e));
    if ((e = g->lanes[i].create()) != cudaSuccess) return fail(static_cast<int>(e));
    if ((e = cudaMalloc(reinterpret_cast<void**>(&g->status[i]), sizeof(int))) != cudaSuccess)
      return fail(static_cast<int>(e));
    if ((e = cudaMemset(g->status[i], 0, sizeof(int))) != cudaSuccess)
      return fail(static_cast<int>(e));
    cudaError_t ie;
    const DeviceInfo* di = current_device_info(&ie);
    if (!di) return fail(static_cast<int>(ie));
    g->workspace_bytes[i] = umma_stream_k_workspace(di->sm_count);
    if ((e = cudaMalloc(&g->workspace[i], g->workspace_bytes[i])) != cudaSuccess)
      return fail(static_cast<int>(e));
  }
  *out = g;
  return TFCCB200_OK;
}

int tfccb200_group_destroy(tfccb200_group* g) {
  if (!g) return TFCCB200_EINVAL;
  DeviceScope scope;
  for (int i = 0; i < g->ndev; ++i) {
    if (cudaSetDevice(g->dev[i]) != cudaSuccess) continue;
    if (g->stream[i]) cudaStreamSynchronize(g->stream[i]);
    if (g->A[i]) cudaFree(g->A[i]);
    if (g->B[i]) cudaFree(g->B[i]);
    if (g->C[i]) cudaFree(g->C[i]);
    if (g->workspace[i]) cudaFree(g->workspace[i]);
    if (g->status[i]) cudaFree(g->status[i]);
    if (g->done[i]) cudaEventDestroy(g->done[i]);
    g->lanes[i].destroy();
    if (g->stream[i]) cudaStreamDestroy(g->stream[i]);
  }
  delete g;
  return TFCCB200_OK;
}

int tfccb200_group_size(const tfccb200_group* g) { return g ? g->ndev : 0; }

int tfccb200_group_device(const tfccb200_group* g, int member) {
  return (g && member >= 0 && member < g->ndev) ? g->dev[member] : -1;
}

void* tfccb200_group_stream(const tfccb200_group* g, int member) {
  return (g && member >= 0 && member < g->ndev) ? g->stream[member] : nullptr;
}

int tfccb200_group_sync(tfccb200_group* g) {
  if (!g) return TFCCB200_EINVAL;
  DeviceScope scope;
  return group_finish(g);
}

int tfccb200_group_sgemm_nsplit(tfccb200_group* g, const float* const* A,
                                const float* const* B_shards, float* const* C,
                                const float* const* bias_shards, unsigned M, unsigned N_shard,
                                unsigned K, int precision_mode) {
  if (!g || !A || !B_shards || !C) return TFCCB200_EINVAL;
  DeviceScope scope;
  cudaError_t e;
  // the members' earlier work (e.g. readers of the previous C) is finished before anyone writes
  if ((e = group_barrier(g)) != cudaSuccess) return static_cast<int>(e);
  for (int i = 0; i < g->ndev; ++i) {
    if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return static_cast<int>(e);
    int st = tfccb200_sgemm_nsplit_push(g->stream[i], A[i], B_shards[i], C, g->ndev, i,
                                        bias_shards ? bias_shards[i] : nullptr, M, N_shard, K,
                                        precision_mode, nullptr, g->workspace[i],
                                        g->workspace_bytes[i], g->status[i]);
    if (st != TFCCB200_OK) return st;
  }
  if ((e = group_barrier(g)) != cudaSuccess) return static_cast<int>(e);
  return TFCCB200_OK;
}

int tfccb200_group_qgemm_nsplit(tfccb200_group* g, const uint8_t* const* A,
                                const int32_t* const* rsA, int32_t offA,
                                const int8_t* const* B_shards, const int32_t* const* rsB_shards,
                                int32_t offB, int32_t* const* C, unsigned M, unsigned N_shard,
                                unsigned K) {
  if (!g || !A || !rsA || !B_shards || !rsB_shards || !C) return TFCCB200_EINVAL;
  DeviceScope scope;
  cudaError_t e;
  if ((e = group_barrier(g)) != cudaSuccess) return static_cast<int>(e);
  for (int i = 0; i < g->ndev; ++i) {
    if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return static_cast<int>(e);
    int st = tfccb200_qgemm_nsplit_push(g->stream[i], A[i], rsA[i], offA, B_shards[i],
                                        rsB_shards[i], offB, C, g->ndev, i, M, N_shard, K,
                                        nullptr, g->status[i]);
    if (st != TFCCB200_OK) return st;
  }
  if ((e = group_barrier(g)) != cudaSuccess) return static_cast<int>(e);
  return TFCCB200_OK;
}

int tfccb200_group_sgemm_nsplit_host(tfccb200_group* g, const float* hA, const float* hB,
                                     float* hC, unsigned M, unsigned N, unsigned K,
                                     int precision_mode) {
  if (!g || !hA || !hB || !hC || M == 0 || N == 0 || K == 0) return TFCCB200_EINVAL;
  const unsigned G = static_cast<unsigned>(g->ndev);
  if (M % G != 0 || N % G != 0) return TFCCB200_EINVAL;
  if (static_cast<unsigned long long>(M) * K > 0xffffffffull ||
      static_cast<unsigned long long>(K) * N > 0xffffffffull ||
      static_cast<unsigned long long>(M) * N > 0xffffffffull)
    return TFCCB200_EOVERFLOW;
  const unsigned ns = N / G, rows = M / G;
  DeviceScope scope;
  cudaError_t e;
  const size_t need_a = static_cast<size_t>(M) * K, need_b = static_cast<size_t>(K) * ns,
               need_c = static_cast<size_t>(M) * N;
  if (need_a > g->a_elems || need_b > g->b_elems || need_c > g->c_elems) {
    int st = group_finish(g);  // nobody may still use the buffers that are replaced
    if (st != TFCCB200_OK) return st;
    for (unsigned i = 0; i < G; ++i) {
      if ((e = cudaSetDevice(g->dev[i])) != cudaSuccess) return static_cast<int>(e);
      if (need_a > g->a_elems && (e = grow(&g->A[i], need_a)) != cudaSuccess) return static_cast<int>(e);
      if (need_b > g->b_elems && (e = grow(&g->B[i], need_b)) != cudaSuccess) return static_cast<int>(e);
      if (need_c > g->c_elems && (e = grow(&g->C[i], need_c)) != cudaSuccess) return static_cast<int>(e);
    }
    g->a_elems = std::max(g->a_elems, need_a);
    g->b_elems = std::max(g->b_elems, need_b);
    g->c_elems = std::max(g->c_elems, need_c);
  }
  NsplitHostRank r[8] = {};
  for (unsigned i = 0; i < G; ++i) {
    r[i] = {};
    r[i].stream = g->stream[i];
    r[i].lanes = &g->lanes[i];
    r[i].hA_rows = hA + static_cast<size_t>(i) * rows * K;
    r[i].hB_shard = hB + static_cast<size_t>(i) * ns;
    r[i].ldb_host = N;
    r[i].hC_rows = hC + static_cast<size_t>(i) * rows * N;
    r[i].A_ranks = g->A;
    r[i].B_shard_dev = g->B[i];
    r[i].C_ranks = g->C;
    r[i].num_ranks = G; r[i].rank = i;
    r[i].M = M; r[i].N_shard = ns; r[i].K = K;
    r[i].precision = precision_mode;
    r[i].workspace = g->workspace[i];
    r[i].workspace_bytes = g->workspace_bytes[i];
    r[i].status = g->status[i];
    int st = nsplit_host_check(r[i]);
    if (st != TFCCB200_OK) return st;
  }
  // whatever happens, no copy from / into the caller's host buffers outlives the call
  struct JoinAll {
    tfccb200_group* g;
    ~JoinAll() {
      for (int i = 0; i < g->ndev; ++i) {
        if (cudaSetDevice(g->dev[i]) != cudaSuccess) continue;
        g->lanes[i].join();
        cudaStreamSynchronize(g->stream[i]);
      }
    }
  } join_all{g};
  const unsigned blocks = nsplit_host_blocks(r[0]);
  auto each = [&](auto&& phase) -> int {
    for (unsigned i = 0; i < G; ++i) {
      cudaError_t ce = cudaSetDevice(g->dev[i]);
      if (ce != cudaSuccess) return static_cast<int>(ce);
      int st = phase(r[i]);
      if (st != TFCCB200_OK) return st;
    }
    return TFCCB200_OK;
  };
  int st = each([&](const NsplitHostRank& x) { return nsplit_host_start(x, blocks); });
  if (st != TFCCB200_OK) return st;
  for (unsigned p = 0; p <= blocks; ++p) {
    st = each([&](const NsplitHostRank& x) { return nsplit_host_before_barrier(x, blocks, p); });
    if (st != TFCCB200_OK) return st;
    if ((e = group_barrier(g)) != cudaSuccess) return static_cast<int>(e);
    st = each([&](const NsplitHostRank& x) { return nsplit_host_after_barrier(x, blocks, p); });
    if (st != TFCCB200_OK) return st;
  }
  return group_finish(g);
}

int tfccb200_sgemm_nsplit_host(void* stream, const float* hA_rows, const float* hB_shard,
                               unsigned ldb_host, float* hC_rows, float* const* A_ranks,
                               float* A_multicast, float* B_shard_dev, float* const* C_ranks,
                               float* C_multicast, unsigned num_ranks, unsigned rank, unsigned M,
                               unsigned N_shard, unsigned K, int precision_mode, void* workspace,
                               size_t workspace_bytes, tfccb200_barrier_fn barrier,
                               void* barrier_ctx, int* device_status) {
  NsplitHostRank r = {};
  r.stream = static_cast<cudaStream_t>(stream);
  r.hA_rows = hA_rows; r.hB_shard = hB_shard; r.ldb_host = ldb_host; r.hC_rows = hC_rows;
  r.A_ranks = A_ranks; r.A_multicast = A_multicast;
  r.B_shard_dev = B_shard_dev;
  r.C_ranks = C_ranks; r.C_multicast = C_multicast;
  r.num_ranks = num_ranks; r.rank = rank;
  r.M = M; r.N_shard = N_shard; r.K = K;
  r.precision = precision_mode;
  r.workspace = workspace; r.workspace_bytes = workspace ? workspace_bytes : 0;
  r.status = device_status;
  if (num_ranks > 1 && !barrier) return TFCCB200_EINVAL;
  int st = nsplit_host_check(r);
  if (st != TFCCB200_OK) return st;
  cudaError_t e;
  HostLanes* lanes = thread_lanes(&e);
  if (!lanes) return static_cast<int>(e);
  r.lanes = lanes;
  // an early return must not leave copies from / into the caller's host buffers in flight
  struct Join {
    HostLanes* l;
    cudaStream_t s;
    ~Join() {
      l->join();
      cudaStreamSynchronize(s);
    }
  } join{lanes, r.stream};
  const unsigned blocks = nsplit_host_blocks(r);
  if ((st = nsplit_host_start(r, blocks)) != TFCCB200_OK) return st;
  for (unsigned p = 0; p <= blocks; ++p) {
    if ((st = nsplit_host_before_barrier(r, blocks, p)) != TFCCB200_OK) return st;
    if (num_ranks > 1 && (st = barrier(barrier_ctx, stream)) != 0) return st;
    if ((st = nsplit_host_after_barrier(r, blocks, p)) != TFCCB200_OK) return st;
  }
  e = cudaStreamSynchronize(r.stream);
  return e == cudaSuccess ? TFCCB200_OK : static_cast<int>(e);
}

}  // extern "C"
