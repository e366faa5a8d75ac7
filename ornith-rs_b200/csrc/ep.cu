// Expert-parallel sparse MoE block: the 256 experts are split evenly over the ranks of one node
// (expert e lives on rank e / (E / world)), token rows stay with the rank that owns their
// sequence, and one layer costs one small exchange each way over NVLink.  The exchanges are the
// library's own kernels over peer memory: every rank maps the others' exchange windows (CUDA IPC),
// stores its rows straight into them with plain stores and raises a flag there; a rank goes on when
// the flags of all its peers have reached the call's sequence number (bounded wait, error flag).
// A decode batch moves a few hundred KB per layer, so the exchange is latency, not bandwidth: two
// kernels per layer instead of NCCL's two grouped collectives (about 40 us each among 8 ranks).
// NCCL remains for the set-up (window handles) and as the exchange when the windows cannot be mapped
// (ORN_EP_NCCL=1 forces it).  No multicast loads, no TMA from peer memory.
//
// The reference is single-GPU (README.md:217-221); what it has is the block this distributes,
// sparse_moe_block (src/ops/moe.rs:662-741), and the building block an expert owner needs: rows
// counting-sorted by expert and each expert run once over its rows (counting_sort +
// switch_glu_rows, src/ops/moe.rs:283-314,463-508, kernels/moe.metal:329-462).
//
// One call, R local rows, nothing read back to the host in between:
//   home   router mat-vec, precise softmax, top-k; shared expert and its gate
//   all    all-gather of the [R, k] routing indices and of the [R, H] rows: every rank then holds
//          the whole table and derives, on the device, which routes are its own
//   owner  routes whose expert it owns, counting-sorted by expert; gate / up / SwiGLU / down with
//          the grouped mat-vec (an expert's records are streamed once for all its rows, every
//          row with the one-row arithmetic); results written straight into the return block of
//          the row's home rank
//   all    all-to-all of fixed-size return blocks [R * k, H] (slots a rank does not own are not
//          read by the receiver, so no counts travel and no host round trip is needed)
//   home   each route's row picked from its owner's block, moe_combine in the reference's
//          ascending-slot bfloat16 order, shared expert added
// Every product runs the row-invariant arithmetic of the single-GPU path and the combine runs at
// home in the reference's order, so the output bits do not depend on the number of ranks.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2: the copy already in the process when the
// host program has one, else the system's), so the library has no link-time dependency on it and
// a single-rank block needs no NCCL at all.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <array>
#include <map>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>

#include "fused.h"
#include "orn_internal.h"

namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  const char* (*GetErrorString)(ncclResult_t);
};

NcclApi* nccl_api(std::string* why) {
  static NcclApi api;
  static bool ok = false;
  static std::string err;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) { err = std::string("cannot load libnccl.so.2: ") + dlerror(); return; }
    bool all = true;
    auto sym = [&](const char* n) { void* p = dlsym(h, n); if (!p) { all = false; err = std::string("libnccl lacks ") + n; } return p; };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    ok = all;
  });
  if (!ok && why) *why = err;
  return ok ? &api : nullptr;
}

// routes of every rank -> this rank's local expert index, or "not mine"
__global__ void ep_map_kernel(const uint32_t* all_inds, int routes, int base, int e_local, uint32_t* rhs_local) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= routes) return;
  const int e = (int)all_inds[i] - base;
  rhs_local[i] = (e >= 0 && e < e_local) ? (uint32_t)e : 0xFFFFFFFFu;
}
// ep_map + counting sort of the routes in one launch of one CTA (a decode batch has a few thousand routes
// at most): seg[e] = first sorted position of local expert e, seg[e_local] = routes this rank owns,
// perm[p] = route at sorted position p; inside an expert the routes keep their order (counting_sort,
// src/ops/moe.rs:463-508).  Passes of 1024 routes: a warp counts its 32 routes per expert, a scan over
// the warps gives every warp its offset inside the expert, the rank inside the warp is a match mask.
constexpr int kRouteMaxLocal = 256;   // local experts the one-launch form handles
constexpr int kRouteMaxRoutes = 8192;
__global__ void __launch_bounds__(1024) ep_route_kernel(const uint32_t* all_inds, int routes, int base, int e_local,
                                                        int* seg /*[e_local + 1]*/, uint32_t* perm) {
  __shared__ int s_seg[kRouteMaxLocal + 1];          // exclusive scan of the counts
  __shared__ int s_done[kRouteMaxLocal];             // routes of the expert placed by earlier passes
  __shared__ uint16_t s_cnt[32][kRouteMaxLocal];     // this pass of 1024 routes: routes per (warp, expert), then the warp's offset
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto local = [&](int i) {
    const int e = i < routes ? (int)all_inds[i] - base : -1;
    return (e >= 0 && e < e_local) ? e : -1;
  };
  // totals per expert
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) s_seg[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < routes; i += blockDim.x) {
    const int e = local(i);
    if (e >= 0) atomicAdd(&s_seg[e], 1);
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan, 32 experts per step
    int carry = 0;
    for (int e0 = 0; e0 <= e_local; e0 += 32) {
      const int e = e0 + lane;
      const int c = e < e_local ? s_seg[e] : 0;
      int incl = c;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      if (e <= e_local) s_seg[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) s_done[e] = 0;
  __syncthreads();
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) seg[e] = s_seg[e];
  // stable placement
  for (int i0 = 0; i0 < routes; i0 += blockDim.x) {
    for (int e = lane; e < e_local; e += 32) s_cnt[warp][e] = 0;
    __syncwarp();
    const int i = i0 + threadIdx.x;
    const int e = local(i);
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) s_cnt[warp][e] = (uint16_t)__popc(same);
    __syncthreads();
    for (int x = threadIdx.x; x < e_local; x += blockDim.x) {  // offsets of the warps inside expert x, then its new total
      int acc = s_done[x];
      for (int w = 0; w < 32; ++w) {
        const int c = s_cnt[w][x];
        s_cnt[w][x] = (uint16_t)acc;
        acc += c;
      }
      s_done[x] = acc;
    }
    __syncthreads();
    if (e >= 0) perm[s_seg[e] + s_cnt[warp][e] + rank_in_warp] = (uint32_t)i;
    __syncthreads();
  }
}
// lhs[i] = i / k: the row a route belongs to
__global__ void ep_iota_kernel(uint32_t* lhs, int n, int k) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lhs[i] = (uint32_t)(i / k);
}
// xs[p] = x[lhs[perm[p]]] for the p < *n_rows sorted rows this rank owns
__global__ void ep_gather_kernel(const bf16_t* x, const uint32_t* lhs, const uint32_t* perm, const int* n_rows, int K,
                                 bf16_t* xs) {
  const int p = blockIdx.x;
  if (p >= *n_rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)lhs[perm[p]] * K);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * K);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}
// SwiGLU of the owned sorted rows only
__global__ void ep_swiglu_kernel(const bf16_t* g, const bf16_t* u, const int* n_rows, int I, bf16_t* out) {
  const size_t n = (size_t)(*n_rows) * I;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = f2bf(orn_swiglu_bf(bf2f(g[i]), bf2f(u[i])));
}
// home: route j's row comes from the block its owner sent
__global__ void ep_select_kernel(const bf16_t* recv, const uint32_t* inds, int e_local, int blk_rows, int H, bf16_t* ey) {
  const int j = blockIdx.x;
  const int owner = (int)inds[j] / e_local;
  const uint4* src = reinterpret_cast<const uint4*>(recv + ((size_t)owner * blk_rows + j) * H);
  uint4* dst = reinterpret_cast<uint4*>(ey + (size_t)j * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}


// ---- the exchange over peer memory ---------------------------------------------------------------
constexpr int kEpMaxPeers = 8;
constexpr unsigned kEpSpinLimit = 1u << 22;  // polls with a 200 ns sleep between them: a few seconds, then the error flag
struct EpPeers {
  uint8_t* win[kEpMaxPeers];  // exchange window of every rank, as mapped into this process
};
// The last CTA of a grid to get here (its stores and everybody else's are fenced) tells every peer that
// this rank's part of call number `epoch` is in place, then waits until all peers have said the same.
// sync[0] = arrivals of this grid, sync[1] = calls so far (both in this rank's own memory).
ORN_D void ep_signal_and_wait(const EpPeers& peers, int W, int rank, size_t off_flags, int* sync, int* err) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&sync[0], 1) == (int)(gridDim.x * gridDim.y) - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  __threadfence_system();
  const int epoch = sync[1] + 1;
  const int lane = threadIdx.x;
  if (lane < W) {
    volatile int* theirs = reinterpret_cast<volatile int*>(peers.win[lane] + off_flags) + rank;
    *theirs = epoch;
  }
  if (lane < W) {
    volatile int* mine = reinterpret_cast<volatile int*>(peers.win[rank] + off_flags) + lane;
    unsigned spins = 0;
    while (*mine - epoch < 0) {
      if (++spins > kEpSpinLimit) { atomicExch(err, 1); break; }
      __nanosleep(200);
    }
  }
  __syncwarp();
  __threadfence_system();
  if (lane == 0) { sync[0] = 0; sync[1] = epoch; }
}
// all-gather by stores: this rank's R rows and R * k routing indices into slot `rank` of every window
__global__ void __launch_bounds__(256) ep_push_kernel(EpPeers peers, int W, int rank, const bf16_t* x, const uint32_t* inds,
                                                      int R, int H, int k, size_t off_x, size_t off_inds, size_t off_flags,
                                                      int* sync, int* err) {
  const int d = blockIdx.y;
  const size_t nx = (size_t)R * H / 8;
  uint4* dx = reinterpret_cast<uint4*>(peers.win[d] + off_x) + (size_t)rank * nx;
  const uint4* sx = reinterpret_cast<const uint4*>(x);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nx; i += (size_t)gridDim.x * blockDim.x) dx[i] = sx[i];
  if (blockIdx.x == 0) {
    uint32_t* di = reinterpret_cast<uint32_t*>(peers.win[d] + off_inds) + (size_t)rank * R * k;
    for (int i = threadIdx.x; i < R * k; i += blockDim.x) di[i] = inds[i];
  }
  ep_signal_and_wait(peers, W, rank, off_flags, sync, err);
}
// the return: sorted row p of this rank is route perm[p] of the whole table = slot (route mod blk) of the
// expert outputs of home rank (route / blk); the row goes straight to its place there
__global__ void __launch_bounds__(256) ep_return_kernel(EpPeers peers, int W, int rank, const bf16_t* ret, const uint32_t* perm,
                                                        const int* n_owned, int blk, int H, size_t off_ey, size_t off_flags,
                                                        int* sync, int* err) {
  const int n = *n_owned;
  for (int p = blockIdx.x; p < n; p += gridDim.x) {
    const int route = (int)perm[p];
    const int d = route / blk, j = route - d * blk;
    const uint4* src = reinterpret_cast<const uint4*>(ret + (size_t)route * H);
    uint4* dst = reinterpret_cast<uint4*>(peers.win[d] + off_ey) + (size_t)j * (H / 8);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
  }
  ep_signal_and_wait(peers, W, rank, off_flags, sync, err);
}

}  // namespace

// scratch for one shape (R, H, E, k, I, SI)
struct EpBufs {
  bf16_t *gates, *probs, *scores, *sg, *su, *sact, *sy, *gs, *all_x, *xs, *eg, *eu, *eact, *ret_send, *ret_recv, *ey;
  uint32_t *inds, *all_inds, *rhs_local, *lhs, *perm;
  int *seg, *seg1;
  void* gemm_scratch;
  // the exchange over peer memory: all_x, all_inds and ey then live in this rank's window at these offsets
  // (the same on every rank), flags = [2][world] call numbers (gather, return), sync = [2][2] local counters
  bool p2p = false;
  size_t off_x = 0, off_inds = 0, off_ey = 0, off_flags = 0;
  int* sync = nullptr;
};
struct EpSet {
  EpBufs bufs{};
  std::vector<void*> allocs;
};
struct orn_ep : EpBufs {
  orn_ctx* ctx = nullptr;
  int rank = 0, world = 1;
  bool exact = false;  // routed experts through the row-invariant grouped mat-vec instead of the tensor cores
  ncclComm_t comm = nullptr;
  // exchange windows (one per rank, mapped into every process of the group); null = NCCL exchanges
  uint8_t* win = nullptr;
  size_t win_bytes = 0, win_used = 0;
  EpPeers peers{};
  std::vector<void*> peer_maps;  // what cudaIpcOpenMemHandle returned, to close
  // One scratch set per shape a caller has used, kept until the group is destroyed: a caller may
  // have captured a call into a CUDA graph, whose kernel arguments are these addresses.
  std::map<std::array<size_t, 6>, EpSet> sets;
};

namespace {

int ep_reserve(orn_ep* ep, int R, int H, int E, int k, int I, int SI) {
  const std::array<size_t, 6> key = {(size_t)R, (size_t)H, (size_t)E, (size_t)k, (size_t)I, (size_t)SI};
  auto it = ep->sets.find(key);
  if (it != ep->sets.end()) {
    static_cast<EpBufs&>(*ep) = it->second.bufs;
    return ORN_OK;
  }
  orn_ctx* ctx = ep->ctx;
  if (ep->sets.size() >= 64) ORN_FAIL(ctx, ORN_ERR_ALLOC, "ep: more than 64 distinct block shapes on one group");
  const size_t W = ep->world, G = W * R, routes = G * k, el = (size_t)E / W;
  EpSet set;
  EpBufs& b = set.bufs;
  int rc = ORN_OK;
  auto A = [&](auto** p, size_t n) {
    if (rc != ORN_OK) return;
    void* d = nullptr;
    rc = orn_alloc(ctx, sizeof(**p) * (n ? n : 1), &d);
    if (rc == ORN_OK) { set.allocs.push_back(d); *p = (std::remove_reference_t<decltype(**p)>*)d; }
  };
  A(&b.gates, (size_t)R * E); A(&b.probs, (size_t)R * E); A(&b.scores, (size_t)R * k); A(&b.inds, (size_t)R * k);
  A(&b.sg, (size_t)R * SI); A(&b.su, (size_t)R * SI); A(&b.sact, (size_t)R * SI); A(&b.sy, (size_t)R * H); A(&b.gs, (size_t)R);
  // the exchanged buffers: in this rank's window when the group has one (the same offsets on every rank:
  // all ranks reserve the same shapes in the same order, as the collectives they replace already require)
  auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t need_win = up256(G * H * sizeof(bf16_t)) + up256(routes * sizeof(uint32_t)) + up256((size_t)R * k * H * sizeof(bf16_t)) + 256;
  b.p2p = ep->win != nullptr && ep->win_used + need_win <= ep->win_bytes;
  if (b.p2p) {
    size_t o = ep->win_used;
    b.off_x = o; o += up256(G * H * sizeof(bf16_t));
    b.off_inds = o; o += up256(routes * sizeof(uint32_t));
    b.off_ey = o; o += up256((size_t)R * k * H * sizeof(bf16_t));
    b.off_flags = o; o += 256;   // [2][world <= 8] ints, zero since the window was made
    ep->win_used = o;
    b.all_x = reinterpret_cast<bf16_t*>(ep->win + b.off_x);
    b.all_inds = reinterpret_cast<uint32_t*>(ep->win + b.off_inds);
    b.ey = reinterpret_cast<bf16_t*>(ep->win + b.off_ey);
    A(&b.sync, (size_t)4);
    if (rc == ORN_OK) rc = cudaMemset(b.sync, 0, 4 * sizeof(int)) == cudaSuccess ? ORN_OK : ORN_ERR_CUDA;
  } else {
    A(&b.all_inds, routes); A(&b.all_x, G * H); A(&b.ey, (size_t)R * k * H);
  }
  A(&b.rhs_local, routes); A(&b.lhs, routes); A(&b.perm, routes);
  A(&b.seg, 2 * el + 4); A(&b.seg1, (size_t)2);
  A(&b.xs, routes * H); A(&b.eg, routes * I); A(&b.eu, routes * I); A(&b.eact, routes * I);
  A(&b.ret_send, routes * H);
  if (!b.p2p) A(&b.ret_recv, routes * H);
  if (rc == ORN_OK) {
    const size_t big = std::max(qgemm_scratch_bytes((int)routes, (int)el, H), qgemm_scratch_bytes((int)routes, (int)el, I));
    rc = orn_alloc(ctx, big, &b.gemm_scratch);
    if (rc == ORN_OK) set.allocs.push_back(b.gemm_scratch);
  }
  const int seg1[2] = {0, R};
  if (rc == ORN_OK) rc = orn_upload(ctx, b.seg1, seg1, sizeof seg1);
  if (rc == ORN_OK) {
    ep_iota_kernel<<<(unsigned)((routes + 255) / 256), 256, 0, ctx->stream>>>(b.lhs, (int)routes, k);
    rc = orn_launch_check(ctx, "ep_iota");
  }
  if (rc == ORN_OK) rc = orn_sync(ctx);
  if (rc != ORN_OK) {
    for (void* p : set.allocs) cudaFree(p);
    return rc;
  }
  static_cast<EpBufs&>(*ep) = set.bufs;
  ep->sets.emplace(key, std::move(set));
  return ORN_OK;
}

// One window per rank, zeroed, its IPC handle gathered over NCCL, every peer's window mapped here.  Every
// rank takes part in the gathers whatever happened to it before, and the group uses the windows only if
// every rank mapped all of them (a flag gathered the same way), so the ranks always agree.
constexpr size_t kEpWindowBytes = (size_t)96 << 20;
void ep_map_windows(orn_ep* ep, NcclApi* api) {
  orn_ctx* ctx = ep->ctx;
  const int W = ep->world;
  struct Slot { cudaIpcMemHandle_t h; int ok; int pad[15]; };
  static_assert(sizeof(Slot) == 128, "one gathered slot");
  Slot mine{};
  uint8_t* win = nullptr;
  mine.ok = cudaMalloc((void**)&win, kEpWindowBytes) == cudaSuccess && cudaMemset(win, 0, kEpWindowBytes) == cudaSuccess &&
            cudaDeviceSynchronize() == cudaSuccess && cudaIpcGetMemHandle(&mine.h, win) == cudaSuccess;
  Slot* dev = nullptr;
  std::vector<Slot> all(W);
  bool gathered = cudaMalloc((void**)&dev, sizeof(Slot) * (W + 1)) == cudaSuccess;
  auto gather = [&]() {  // mine -> all, over NCCL on the context's stream
    if (!gathered) return false;
    if (cudaMemcpyAsync(dev + W, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return false;
    if (api->AllGather(dev + W, dev, sizeof(Slot), ncclChar, ep->comm, ctx->stream) != ncclSuccess) return false;
    if (cudaMemcpyAsync(all.data(), dev, sizeof(Slot) * W, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) return false;
    return cudaStreamSynchronize(ctx->stream) == cudaSuccess;
  };
  bool ok = gather();
  for (int r = 0; ok && r < W; ++r) ok = all[r].ok != 0;
  std::vector<void*> maps;
  EpPeers peers{};
  for (int r = 0; ok && r < W; ++r) {
    if (r == ep->rank) { peers.win[r] = win; continue; }
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, all[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ok = false; cudaGetLastError(); break; }
    maps.push_back(p);
    peers.win[r] = static_cast<uint8_t*>(p);
  }
  mine.ok = ok ? 1 : 0;   // second round: did everybody map everything?
  bool all_ok = gather();
  for (int r = 0; all_ok && r < W; ++r) all_ok = all[r].ok != 0;
  if (dev) cudaFree(dev);
  if (all_ok) {
    ep->win = win; ep->win_bytes = kEpWindowBytes; ep->win_used = 0; ep->peers = peers; ep->peer_maps = maps;
    return;
  }
  for (void* p : maps) cudaIpcCloseMemHandle(p);
  if (win) cudaFree(win);
  cudaGetLastError();
}

#define EP_NCCL(ctx, api, call)                                                              \
  do {                                                                                       \
    ncclResult_t r__ = (call);                                                               \
    if (r__ != ncclSuccess) {                                                                \
      (ctx)->err = std::string(#call) + ": " + (api)->GetErrorString(r__);                   \
      return ORN_ERR_CUDA;                                                                   \
    }                                                                                        \
  } while (0)

}  // namespace

extern "C" {

int32_t orn_ep_unique_id(uint8_t* id_out) {
  if (!id_out) return ORN_ERR_ARG;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  std::string why;
  NcclApi* api = nccl_api(&why);
  if (!api) return ORN_ERR_STATE;
  ncclUniqueId id;
  if (api->GetUniqueId(&id) != ncclSuccess) return ORN_ERR_CUDA;
  memcpy(id_out, &id, sizeof id);
  return ORN_OK;
}

int32_t orn_ep_init(orn_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world, int32_t flags, orn_ep** out) {
  if (!ctx || !out || world < 1 || rank < 0 || rank >= world) return ORN_ERR_ARG;
  *out = nullptr;
  orn_ep* ep = new orn_ep();
  ep->ctx = ctx; ep->rank = rank; ep->world = world;
  ep->exact = (flags & ORN_EP_EXACT) != 0;
  if (world > 1) {
    if (!id) { delete ep; ORN_FAIL(ctx, ORN_ERR_ARG, "ep_init: more than one rank needs the unique id of rank 0"); }
    std::string why;
    NcclApi* api = nccl_api(&why);
    if (!api) { delete ep; ORN_FAIL(ctx, ORN_ERR_STATE, "ep_init: " + why); }
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    cudaSetDevice(ctx->device);
    ncclResult_t r = api->CommInitRank(&ep->comm, world, uid, rank);
    if (r != ncclSuccess) {
      delete ep;
      ORN_FAIL(ctx, ORN_ERR_CUDA, std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    }
    // exchange windows over peer memory; on any failure the group keeps NCCL for its exchanges
    const char* force = getenv("ORN_EP_NCCL");
    if (world <= kEpMaxPeers && !(force && force[0] == '1')) ep_map_windows(ep, api);
  }
  *out = ep;
  return ORN_OK;
}

int32_t orn_debug_ep_wait_probe(orn_ctx* ctx) {
  if (!ctx) return ORN_ERR_ARG;
  // a window in which rank 0's flag gets written and rank 1's never does; no rows to move
  uint8_t* win = nullptr;
  int* sync = nullptr;
  ORN_CHECK_CUDA(ctx, cudaMalloc((void**)&win, 4096));
  if (cudaMalloc((void**)&sync, 4 * sizeof(int)) != cudaSuccess) { cudaFree(win); ORN_FAIL(ctx, ORN_ERR_ALLOC, "ep wait probe: out of memory"); }
  cudaMemsetAsync(win, 0, 4096, ctx->stream);
  cudaMemsetAsync(sync, 0, 4 * sizeof(int), ctx->stream);
  EpPeers peers{};
  peers.win[0] = win; peers.win[1] = win;
  ep_push_kernel<<<dim3(1, 2), 256, 0, ctx->stream>>>(peers, 2, 0, reinterpret_cast<const bf16_t*>(win),
                                                      reinterpret_cast<const uint32_t*>(win), 0, 8, 1, 1024, 2048, 3072, sync,
                                                      ctx->dev_err);
  int rc = orn_launch_check(ctx, "ep_push");
  cudaStreamSynchronize(ctx->stream);   // the kernel has given up by now; the error flag stays for orn_sync
  cudaFree(win);
  cudaFree(sync);
  return rc;
}

int32_t orn_ep_world(const orn_ep* ep) { return ep ? ep->world : 0; }
int32_t orn_ep_rank(const orn_ep* ep) { return ep ? ep->rank : -1; }
int32_t orn_ep_peer_windows(const orn_ep* ep) { return ep && ep->win != nullptr ? 1 : 0; }

int32_t orn_ep_destroy(orn_ep* ep) {
  if (!ep) return ORN_OK;
  cudaStreamSynchronize(ep->ctx->stream);
  if (ep->comm) {
    NcclApi* api = nccl_api(nullptr);
    if (api) api->CommDestroy(ep->comm);
  }
  for (auto& kv : ep->sets)
    for (void* p : kv.second.allocs) cudaFree(p);
  // every rank leaves its peers' windows before anybody frees one: the caller destroys the groups of
  // all ranks together, and a window is only stored to inside a block call
  for (void* p : ep->peer_maps) cudaIpcCloseMemHandle(p);
  if (ep->win) cudaFree(ep->win);
  delete ep;
  return ORN_OK;
}

int32_t orn_ep_moe_block(orn_ep* ep, const orn_linear* gate, const orn_linear* sw_gate, const orn_linear* sw_up,
                         const orn_linear* sw_down, const orn_linear* sh_gate, const orn_linear* sh_up,
                         const orn_linear* sh_down, const orn_linear* sh_egate, const uint16_t* dev_x, int32_t R,
                         int32_t top_k, int32_t norm_topk, uint16_t* dev_out, uint32_t* dev_inds_out) {
  if (!ep || !gate || !sw_gate || !sw_up || !sw_down || !sh_gate || !sh_up || !sh_down || !sh_egate || !dev_x || !dev_out)
    return ORN_ERR_ARG;
  orn_ctx* ctx = ep->ctx;
  cudaStream_t s = ctx->stream;
  const int W = ep->world, H = gate->K, E = gate->O, I = sw_gate->O, SI = sh_gate->O, k = top_k;
  if (R < 1 || k < 1 || k > E) ORN_FAIL(ctx, ORN_ERR_ARG, "ep_moe_block: bad row count or top_k");
  if (E % W) ORN_FAIL(ctx, ORN_ERR_ARG, "ep_moe_block: the experts do not split evenly over the ranks");
  const int el = E / W;
  if (sw_gate->E != el || sw_up->E != el || sw_down->E != el || sw_gate->K != H || sw_up->K != H || sw_up->O != I ||
      sw_down->O != H || sw_down->K != I || sh_up->O != SI || sh_gate->K != H || sh_up->K != H || sh_down->O != H ||
      sh_down->K != SI || sh_egate->O != 1 || sh_egate->K != H || H % 8)
    ORN_FAIL(ctx, ORN_ERR_ARG, "ep_moe_block: inconsistent weight shapes (routed matrices hold this rank's E / world experts)");
  int rc = ep_reserve(ep, R, H, E, k, I, SI);
  if (rc != ORN_OK) return rc;
  const int G = W * R, routes = G * k, blk = R * k;
  NcclApi* api = W > 1 ? nccl_api(nullptr) : nullptr;
  if (W > 1 && !api) ORN_FAIL(ctx, ORN_ERR_STATE, "ep_moe_block: NCCL is not loaded");
#define EPCK(call) do { int rc__ = (call); if (rc__ != ORN_OK) return rc__; } while (0)
  // ---- home: routing and the shared expert (one launch per matrix over all R rows)
  uint32_t* inds = dev_inds_out ? dev_inds_out : ep->inds;
  // the router and the shared expert's gate in one launch (neither depends on the exchange)
  EPCK(k_grouped_gemv2(ctx, s, gate, ep->gates, sh_egate, ep->gs, dev_x, ep->seg1, R));
  if (E <= 512) {
    EPCK(k_softmax_topk(ctx, s, ep->gates, R, E, k, inds, ep->scores));
  } else {
    EPCK(k_softmax_precise(ctx, s, ep->gates, R, E, ep->probs));
    EPCK(k_router_topk(ctx, s, ep->probs, R, E, k, inds, ep->scores));
  }
  // ---- every rank learns the whole routing table and the rows
  const uint32_t* all_inds = inds;
  const bf16_t* all_x = dev_x;
  if (W > 1 && ep->p2p) {
    ep_push_kernel<<<dim3(4, W), 256, 0, s>>>(ep->peers, W, ep->rank, dev_x, inds, R, H, k, ep->off_x, ep->off_inds, ep->off_flags,
                                             ep->sync, ctx->dev_err);
    EPCK(orn_launch_check(ctx, "ep_push"));
    all_inds = ep->all_inds;
    all_x = ep->all_x;
  } else if (W > 1) {
    EP_NCCL(ctx, api, api->GroupStart());
    EP_NCCL(ctx, api, api->AllGather(inds, ep->all_inds, (size_t)R * k, ncclUint32, ep->comm, s));
    EP_NCCL(ctx, api, api->AllGather(dev_x, ep->all_x, (size_t)R * H, ncclBfloat16, ep->comm, s));
    EP_NCCL(ctx, api, api->GroupEnd());
    ctx->launches += 2;
    all_inds = ep->all_inds;
    all_x = ep->all_x;
  }
  // The shared expert depends on the block's input only: on the tensor-core path its three launches run on
  // the context's side stream beside the routed chain (forked here, joined before the combine; inside a
  // captured step the two become parallel branches of the graph).  With few rows per rank every kernel of
  // the block is a short latency chain and the SMs are mostly idle, so the two chains overlap.
  const bool side = !ep->exact && orn_side_stream(ctx);
  cudaStream_t ss = side ? ctx->side : s;
  if (side) {
    ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev_fork, s));
    ORN_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
  }
  const bool wide_shared = !ep->exact && R >= 16 && H % 64 == 0 && SI % 64 == 0;
  if (wide_shared) {  // like the routed experts: one dense contraction per matrix over all R rows
    if (sh_gate->kind == sh_up->kind && sh_gate->K == sh_up->K) {  // one launch for both (a row's bits do not depend on the tile shape)
      const orn_linear* pl[2] = {sh_gate, sh_up};
      void* py[2] = {ep->sg, ep->su};
      const int ld[2] = {SI, SI};
      EPCK(f_qgemm_multi(ctx, ss, pl, py, ld, 2, dev_x, R));
    } else {
      EPCK(f_qgemm(ctx, ss, sh_gate, dev_x, R, ep->sg, SI, nullptr, nullptr));
      EPCK(f_qgemm(ctx, ss, sh_up, dev_x, R, ep->su, SI, nullptr, nullptr));
    }
  } else {
    EPCK(k_grouped_gemv(ctx, s, sh_gate, dev_x, ep->seg1, ep->sg, nullptr, R));
    EPCK(k_grouped_gemv(ctx, s, sh_up, dev_x, ep->seg1, ep->su, nullptr, R));
  }
  // the shared expert's SwiGLU and down projection: with the routed experts' (one launch for both SwiGLUs)
  // on the tensor-core path, right here otherwise
  const bool joint_swiglu = !ep->exact && !side;
  if (!joint_swiglu) {
    EPCK(k_swiglu(ctx, ss, ep->sg, ep->su, R * SI, ep->sact));
    if (wide_shared) EPCK(f_qgemm(ctx, ss, sh_down, ep->sact, R, ep->sy, H, nullptr, nullptr));
    else EPCK(k_grouped_gemv(ctx, ss, sh_down, ep->sact, ep->seg1, ep->sy, nullptr, R));
  }
  if (side) ORN_CHECK_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->side));
  // ---- owner: this rank's routes, sorted by expert
  if (el <= kRouteMaxLocal && routes <= kRouteMaxRoutes) {
    ep_route_kernel<<<1, 1024, 0, s>>>(all_inds, routes, ep->rank * el, el, ep->seg, ep->perm);
    EPCK(orn_launch_check(ctx, "ep_route"));
  } else {
    ep_map_kernel<<<(routes + 255) / 256, 256, 0, s>>>(all_inds, routes, ep->rank * el, el, ep->rhs_local);
    EPCK(orn_launch_check(ctx, "ep_map"));
    EPCK(f_route_sort(ctx, s, ep->rhs_local, routes, el, ep->seg, ep->seg + el + 1, ep->perm));
  }
  const int* n_owned = ep->seg + el;  // device: seg[el] = number of routes this rank owns
  ep_gather_kernel<<<routes, 128, 0, s>>>(all_x, ep->lhs, ep->perm, n_owned, H, ep->xs);
  EPCK(orn_launch_check(ctx, "ep_gather"));
  // sorted row p is route perm[p] of the whole table = slot perm[p] of the return blocks laid end to end
  bf16_t* ret = W > 1 ? ep->ret_send : ep->ey;
  if (ep->exact) {
    EPCK(k_grouped_gemv(ctx, s, sw_gate, ep->xs, ep->seg, ep->eg, nullptr, routes));
    EPCK(k_grouped_gemv(ctx, s, sw_up, ep->xs, ep->seg, ep->eu, nullptr, routes));
    ep_swiglu_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ep->eg, ep->eu, n_owned, I, ep->eact);
    EPCK(orn_launch_check(ctx, "ep_swiglu"));
    EPCK(k_grouped_gemv(ctx, s, sw_down, ep->eact, ep->seg, ret, ep->perm, routes));
  } else {
    // a decode batch of many sequences is a dense contraction per expert: the grouped tensor-core
    // product (an expert's records dequantised once per tile for all its rows)
    const int hint = std::max(1, (routes / W) / el);
    QGemmGroup sorted{ep->seg, nullptr, hint}, back{ep->seg, ep->perm, hint};
    if (sw_gate->kind == sw_up->kind) {  // gate and up of every expert in one launch (one plan, one tile space)
      const orn_linear* pl[2] = {sw_gate, sw_up};
      void* py[2] = {ep->eg, ep->eu};
      const int ld[2] = {I, I};
      EPCK(f_qgemm_multi(ctx, s, pl, py, ld, 2, ep->xs, routes, &sorted, ep->gemm_scratch));
    } else {
      EPCK(f_qgemm(ctx, s, sw_gate, ep->xs, routes, ep->eg, I, &sorted, ep->gemm_scratch));
      EPCK(f_qgemm(ctx, s, sw_up, ep->xs, routes, ep->eu, I, &sorted, ep->gemm_scratch));
    }
    if (joint_swiglu) {
      EPCK(k_swiglu2(ctx, s, ep->sg, ep->su, (size_t)R * SI, ep->sact, ep->eg, ep->eu, n_owned, I, ep->eact));
      if (wide_shared) EPCK(f_qgemm(ctx, s, sh_down, ep->sact, R, ep->sy, H, nullptr, nullptr));
      else EPCK(k_grouped_gemv(ctx, s, sh_down, ep->sact, ep->seg1, ep->sy, nullptr, R));
    } else {
      ep_swiglu_kernel<<<ctx->sm_count * 4, 256, 0, s>>>(ep->eg, ep->eu, n_owned, I, ep->eact);
      EPCK(orn_launch_check(ctx, "ep_swiglu"));
    }
    EPCK(f_qgemm(ctx, s, sw_down, ep->eact, routes, ret, H, &back, ep->gemm_scratch));
  }
  // ---- the return: one fixed-size block per pair of ranks
  if (W > 1 && ep->p2p) {
    ep_return_kernel<<<std::min(routes, 2 * ctx->sm_count), 256, 0, s>>>(ep->peers, W, ep->rank, ep->ret_send, ep->perm, n_owned, blk, H,
                                                                         ep->off_ey, ep->off_flags + 32, ep->sync + 2, ctx->dev_err);
    EPCK(orn_launch_check(ctx, "ep_return"));
  } else if (W > 1) {
    const size_t n = (size_t)blk * H;
    EP_NCCL(ctx, api, api->GroupStart());
    for (int d = 0; d < W; ++d) {
      EP_NCCL(ctx, api, api->Send(ep->ret_send + (size_t)d * n, n, ncclBfloat16, d, ep->comm, s));
      EP_NCCL(ctx, api, api->Recv(ep->ret_recv + (size_t)d * n, n, ncclBfloat16, d, ep->comm, s));
    }
    EP_NCCL(ctx, api, api->GroupEnd());
    ctx->launches += 1;
    ep_select_kernel<<<blk, 128, 0, s>>>(ep->ret_recv, inds, el, blk, H, ep->ey);
    EPCK(orn_launch_check(ctx, "ep_select"));
  }
  // ---- home: combine in the reference's order
  if (side) ORN_CHECK_CUDA(ctx, cudaStreamWaitEvent(s, ctx->ev_join, 0));
  EPCK(k_moe_combine(ctx, s, ep->scores, ep->ey, ep->gs, ep->sy, R, k, H, norm_topk, dev_out));
#undef EPCK
  return ORN_OK;
}

}  // extern "C"
