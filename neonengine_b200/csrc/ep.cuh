// Expert parallelism: experts are sharded evenly over the ranks of one node, the router is
// replicated, every rank routes its own tokens.  Two exchanges per pass, both all-to-all-v
// built from grouped ncclSend/ncclRecv over NVLink: token rows (bf16) to the ranks that own
// their experts, and the experts' outputs (fp32) back.  NCCL is loaded with dlopen so the
// single-GPU library has no link-time dependency on it.  Kernels never touch peer memory:
// rows land in this GPU's own receive buffer first.
#pragma once
#include <dlfcn.h>
#include <nccl.h>

namespace neon {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

inline NcclApi& nccl_api() {
    static NcclApi api;
    if (api.lib) return api;
    // RTLD_NOLOAD first: reuse the copy a host framework has already loaded, if any
    api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!api.lib) api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!api.lib) return api;
    bool all = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(api.lib, name);
        if (!p) all = false;
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = all;
    return api;
}

// Exchange plan of one rank from the gathered histograms all_counts[ep_size][n_experts]
// (all_counts[r][e] = entries rank r routes to global expert e).  Rows travel grouped by
// destination rank and, inside a rank's segment, by ascending expert, so the receiver can
// rebuild each row's expert from the counts alone.
//   send_rows[r], send_off[r]: rows this rank sends to r and their start in its sorted order
//   recv_rows[r], recv_off[r]: rows it receives from r and their start in its receive buffer
//   row_expert[i]: LOCAL expert id (0..n_local-1) of received row i (at most cap entries)
// Returns the number of received rows, or -1 when it exceeds cap.
inline int ep_plan(const int32_t* all_counts, int ep_size, int n_experts, int rank, int32_t* send_rows,
                   int32_t* send_off, int32_t* recv_rows, int32_t* recv_off, int32_t* row_expert, int cap) {
    const int nl = n_experts / ep_size, e_lo = rank * nl;
    int so = 0, ro = 0;
    for (int r = 0; r < ep_size; ++r) {
        int s = 0, v = 0;
        for (int e = 0; e < nl; ++e) {
            s += all_counts[(size_t)rank * n_experts + r * nl + e];
            v += all_counts[(size_t)r * n_experts + e_lo + e];
        }
        send_rows[r] = s;
        send_off[r] = so;
        recv_rows[r] = v;
        recv_off[r] = ro;
        so += s;
        if (ro + v > cap) return -1;
        if (row_expert) {
            int i = ro;
            for (int e = 0; e < nl; ++e)
                for (int c = all_counts[(size_t)r * n_experts + e_lo + e]; c > 0; --c) row_expert[i++] = e;
        }
        ro += v;
    }
    return ro;
}

// The receive-capacity verdict of a pass, computed from the gathered histograms alone so that
// every rank reaches the same answer before any row travels: returns the lowest rank whose
// receive total exceeds its capacity caps[r], or -1 when every rank fits.  A rank that decided
// on its own total only would leave its peers waiting in the exchange for rows that never come.
inline int ep_first_overflow(const int32_t* all_counts, int ep_size, int n_experts, const int32_t* caps) {
    const int nl = n_experts / ep_size;
    for (int r = 0; r < ep_size; ++r) {
        long long total = 0;
        for (int src = 0; src < ep_size; ++src)
            for (int e = 0; e < nl; ++e) total += all_counts[(size_t)src * n_experts + r * nl + e];
        if (total > caps[r]) return r;
    }
    return -1;
}

// ---- exchanges by plain stores into the peers' buffers (NVLink peer-to-peer) ----------------------
// With the peers' receive buffers mapped into this process (CUDA IPC), a rank writes the rows it owes
// straight where they belong: token rows into the expert owner's xrecv, expert outputs - from the down
// product's epilogue, tile by tile while the product runs - into the token owner's yrecv.  No copy
// engine, no library kernel and no TMA multicast touches peer memory: only this library's own st.global.
constexpr int kMaxPeerRanks = 8;

// Where the rows of one block go: block b (rows [row_off[b], row_off[b + 1]) of the local order) lands in
// buffer base[b] starting at row dst_off[b].
template <typename T>
struct PeerRows {
    int n_ranks;  // 0 = not in use
    int row_off[kMaxPeerRanks + 1];
    int dst_off[kMaxPeerRanks];
    T* base[kMaxPeerRanks];
};

template <typename T>
__device__ __forceinline__ T* peer_row(const PeerRows<T>& t, int row, int width) {
    int b = 0;
    while (b + 1 < t.n_ranks && row >= t.row_off[b + 1]) ++b;
    return t.base[b] + (size_t)(t.dst_off[b] + row - t.row_off[b]) * width;
}

// Host side of the two tables of one rank, from the gathered histograms.  rows(a -> b) = entries rank a
// routes to rank b's experts.  Dispatch: my sorted rows for rank r start at send_off[r] and land in r's xrecv
// behind the rows of the ranks before me.  Return: received rows from rank r start at recv_off[r] and go
// back into r's yrecv where r's sorted rows for me start.
inline void ep_peer_offsets(const int32_t* all_counts, int ep_size, int n_experts, int rank, int32_t* dispatch_dst_off,
                            int32_t* return_dst_off) {
    const int nl = n_experts / ep_size;
    auto rows = [&](int a, int b) {
        int s = 0;
        for (int e = 0; e < nl; ++e) s += all_counts[(size_t)a * n_experts + b * nl + e];
        return s;
    };
    for (int r = 0; r < ep_size; ++r) {
        int d = 0, b = 0;
        for (int q = 0; q < rank; ++q) {
            d += rows(q, r);   // rows of lower ranks in r's receive buffer
            b += rows(r, q);   // rows r sends to lower ranks, in r's sorted order
        }
        dispatch_dst_off[r] = d;
        return_dst_off[r] = b;
    }
}

// Token rows to the expert owners: sorted entry p -> its place in the owner's xrecv (16-byte vectors).  A fixed
// grid walks the rows, one warp per row, four vectors per lane in flight (the stores cross NVLink: what limits
// them is how many are outstanding); one system-scope fence per CTA, after a CTA barrier, publishes all of its
// stores (a fence per thread costs far more than the copy).
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint16_t* __restrict__ hidden, const int32_t* __restrict__ perm, int k,
                                                           int H, int n, PeerRows<uint16_t> t) {
    const int nvec = H / 8, lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n; p += warps) {
        const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)(perm[p] / k) * H);
        uint4* dst = reinterpret_cast<uint4*>(peer_row(t, p, H));
        for (int i = lane; i < nvec; i += 128) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 32 * j < nvec) v[j] = src[i + 32 * j];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + 32 * j < nvec) dst[i + 32 * j] = v[j];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
}

// xsend[p, :] = hidden[perm[p] / k, :] for the n sorted entries (16-byte vectors).
__global__ void pack_rows_kernel(const uint16_t* __restrict__ hidden, const int32_t* __restrict__ perm, int k, int H, int n,
                                 uint16_t* __restrict__ xsend) {
    const int p = blockIdx.x;
    if (p >= n) return;
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)(perm[p] / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(xsend + (size_t)p * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t, c] = sum over slots s (in order) of w[t*k+s] * y[inv[t*k+s], c].
__global__ void combine_weighted_kernel(const float* __restrict__ y, const int32_t* __restrict__ inv,
                                        const float* __restrict__ w, int T, int H, int k, float* __restrict__ out) {
    const int t = blockIdx.y;
    const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 * 4 >= H) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sl = 0; sl < k; ++sl) {
        const int pos = inv[t * k + sl];
        if (pos < 0) continue;
        const float ws = w[t * k + sl];
        const float4 v = *reinterpret_cast<const float4*>(y + (size_t)pos * H + 4 * c4);
        s.x += ws * v.x; s.y += ws * v.y; s.z += ws * v.z; s.w += ws * v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)t * H + 4 * c4) = s;
}

__global__ void fill_ones_kernel(float* p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 1.f;
}

}  // namespace neon
