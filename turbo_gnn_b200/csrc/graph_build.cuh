// Device-side graph construction: COO -> CSR ordered by (row, column), degree order
// statistics and the light / heavy row partition.
//
// Everything rests on one stable LSD radix sort of 64-bit keys with an optional 32-bit
// payload (8-bit digits, only the passes the key range needs):
//
//   COO -> CSR      key = row * num_nodes + column, payload = input position (optional);
//                   after the sort the column is key % num_nodes and indptr[r] is the lower
//                   bound of r * num_nodes in the sorted keys (one binary search per row, so
//                   runs of empty rows cost nothing special).
//   order stats     key = degree; the sorted array is indexed directly.
//   partition       one 1-bit pass, key = (degree >= cut), payload = row id: the stable
//                   scatter leaves light ids ascending, then heavy ids ascending.
//
// A pass is three kernels: per-CTA digit histogram over the CTA's contiguous key range,
// exclusive scan of the [digit][CTA] table by one CTA, and a scatter in which every CTA
// walks its range tile by tile keeping the running output position of each digit in
// shared memory.  Inside a tile a key's rank among equal digits is its warp's start plus
// the count of earlier equal digits in the warp (match_any per round of 32 keys), which
// keeps the input order, i.e. the sort is stable.  No kernel waits on another.
#pragma once

#include "common.cuh"

namespace tgnn {
namespace gb {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kItems = 8;                          // keys per thread and tile
constexpr int kTile = kSortThreads * kItems;       // keys per tile
constexpr int kRadix = 256;

// ---- keys -----------------------------------------------------------------------------

// key = row * num_nodes + col; an id outside [0, num_nodes) raises *bad and is clamped.
template <typename I>
__global__ void __launch_bounds__(256) pack_edge_keys_kernel(const I *__restrict__ rows, const I *__restrict__ cols,
                                                             int64_t n, uint64_t num_nodes, uint64_t *__restrict__ keys,
                                                             uint32_t *__restrict__ order, int32_t *__restrict__ bad) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t r = static_cast<int64_t>(rows[i]);
        int64_t c = static_cast<int64_t>(cols[i]);
        if (r < 0 || c < 0 || static_cast<uint64_t>(r) >= num_nodes || static_cast<uint64_t>(c) >= num_nodes) {
            *bad = 1;
            r = 0;
            c = 0;
        }
        keys[i] = static_cast<uint64_t>(r) * num_nodes + static_cast<uint64_t>(c);
        if (order != nullptr) order[i] = static_cast<uint32_t>(i);
    }
}

// key = degree of row i (mode 0), or 1 / 0 for float(degree) >= cut (mode 1, payload = i).
template <typename I>
__global__ void __launch_bounds__(256) degree_keys_kernel(const I *__restrict__ indptr, int64_t n_rows, int mode,
                                                          float cut, uint64_t *__restrict__ keys,
                                                          uint32_t *__restrict__ ids) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_rows; i += stride) {
        const int64_t deg = static_cast<int64_t>(indptr[i + 1]) - static_cast<int64_t>(indptr[i]);
        if (mode == 0) {
            keys[i] = static_cast<uint64_t>(deg);
        } else {
            keys[i] = static_cast<float>(deg) >= cut ? 1u : 0u;
            ids[i] = static_cast<uint32_t>(i);
        }
    }
}

// ---- one radix pass -----------------------------------------------------------------------

__global__ void __launch_bounds__(kSortThreads) radix_hist_kernel(const uint64_t *__restrict__ keys, int64_t n,
                                                                  int shift, int64_t tiles_per_cta,
                                                                  uint32_t *__restrict__ hist) {
    __shared__ uint32_t h[kRadix];
    h[threadIdx.x] = 0;
    __syncthreads();
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * tiles_per_cta * kTile;
    int64_t end = begin + tiles_per_cta * kTile;
    if (end > n) end = n;
    for (int64_t i = begin + threadIdx.x; i < end; i += kSortThreads)
        atomicAdd(&h[static_cast<uint32_t>(keys[i] >> shift) & (kRadix - 1)], 1u);
    __syncthreads();
    hist[static_cast<size_t>(threadIdx.x) * gridDim.x + blockIdx.x] = h[threadIdx.x];
}

// In-place exclusive scan of `m` counters by one CTA of 1024 threads.
__global__ void __launch_bounds__(1024) scan_counters_kernel(uint32_t *__restrict__ v, int64_t m) {
    __shared__ uint32_t warp_sum[32];
    const int tid = threadIdx.x;
    const int64_t per = (m + 1023) / 1024;
    const int64_t b = tid * per;
    int64_t e = b + per;
    if (e > m) e = m;
    uint32_t sum = 0;
    for (int64_t i = b; i < e; ++i) sum += v[i];
    // exclusive scan of the 1024 thread sums
    uint32_t incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(kFull, incl, o);
        if ((tid & 31) >= o) incl += up;
    }
    if ((tid & 31) == 31) warp_sum[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        uint32_t w = warp_sum[tid];
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(kFull, wi, o);
            if (tid >= o) wi += up;
        }
        warp_sum[tid] = wi - w;  // exclusive
    }
    __syncthreads();
    uint32_t run = warp_sum[tid >> 5] + incl - sum;
    for (int64_t i = b; i < e; ++i) {
        const uint32_t c = v[i];
        v[i] = run;
        run += c;
    }
}

__global__ void __launch_bounds__(kSortThreads)
    radix_scatter_kernel(const uint64_t *__restrict__ kin, uint64_t *__restrict__ kout, const uint32_t *__restrict__ vin,
                         uint32_t *__restrict__ vout, int64_t n, int shift, int64_t tiles_per_cta,
                         const uint32_t *__restrict__ offs) {
    __shared__ uint32_t base[kRadix];                 // next output position of digit d for this CTA
    __shared__ uint32_t wcnt[kSortWarps][kRadix];     // per-warp digit counts, then per-warp starts
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const unsigned lt_mask = (1u << lane) - 1u;
    base[tid] = offs[static_cast<size_t>(tid) * gridDim.x + blockIdx.x];
    const int64_t cta_begin = static_cast<int64_t>(blockIdx.x) * tiles_per_cta * kTile;
    int64_t cta_end = cta_begin + tiles_per_cta * kTile;
    if (cta_end > n) cta_end = n;
    for (int64_t tile = cta_begin; tile < cta_end; tile += kTile) {
        for (int j = tid; j < kSortWarps * kRadix; j += kSortThreads) (&wcnt[0][0])[j] = 0;
        __syncthreads();
        uint64_t key[kItems];
        uint32_t val[kItems];
        uint32_t rank[kItems];
        const int64_t wbase = tile + static_cast<int64_t>(warp) * (32 * kItems);
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            const int64_t idx = wbase + i * 32 + lane;
            const bool valid = idx < cta_end;
            key[i] = valid ? kin[idx] : 0;
            val[i] = (valid && vin != nullptr) ? vin[idx] : 0;
            const uint32_t d = static_cast<uint32_t>(key[i] >> shift) & (kRadix - 1);
            // lanes past the end get values no other lane has, so they match nobody
            const unsigned peers = __match_any_sync(kFull, valid ? d : (kRadix + lane));
            const int leader = __ffs(peers) - 1;
            uint32_t old = 0;
            if (valid) old = wcnt[warp][d];
            __syncwarp();
            if (valid && lane == leader) wcnt[warp][d] = old + __popc(peers);
            __syncwarp();
            rank[i] = old + __popc(peers & lt_mask);
        }
        __syncthreads();
        {
            uint32_t run = base[tid];
#pragma unroll
            for (int w = 0; w < kSortWarps; ++w) {
                const uint32_t c = wcnt[w][tid];
                wcnt[w][tid] = run;
                run += c;
            }
            base[tid] = run;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
            const int64_t idx = wbase + i * 32 + lane;
            if (idx < cta_end) {
                const uint32_t d = static_cast<uint32_t>(key[i] >> shift) & (kRadix - 1);
                const uint32_t pos = wcnt[warp][d] + rank[i];
                kout[pos] = key[i];
                if (vout != nullptr) vout[pos] = val[i];
            }
        }
        __syncthreads();
    }
}

// ---- CSR from sorted keys ---------------------------------------------------------------------

// indptr[q] = number of keys below q * num_nodes, q = 0 .. num_nodes.
template <typename O>
__global__ void __launch_bounds__(256) indptr_from_keys_kernel(const uint64_t *__restrict__ keys, int64_t n,
                                                               uint64_t num_nodes, O *__restrict__ indptr) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q <= num_nodes; q += stride) {
        const uint64_t target = q * num_nodes;
        int64_t lo = 0, hi = n;
        while (lo < hi) {
            const int64_t mid = lo + ((hi - lo) >> 1);
            if (keys[mid] < target)
                lo = mid + 1;
            else
                hi = mid;
        }
        indptr[q] = static_cast<O>(lo);
    }
}

template <typename O>
__global__ void __launch_bounds__(256) columns_from_keys_kernel(const uint64_t *__restrict__ keys, int64_t n,
                                                                uint64_t num_nodes, O *__restrict__ indices) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        indices[i] = static_cast<O>(keys[i] % num_nodes);
}

template <typename O>
__global__ void __launch_bounds__(256) copy_ids_kernel(const uint32_t *__restrict__ ids, int64_t n, O *__restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = static_cast<O>(ids[i]);
}

// out = { sorted[k_lo], sorted[k_hi], sorted[n - 1] }
__global__ void pick_order_stats_kernel(const uint64_t *__restrict__ sorted, int64_t n, int64_t k_lo, int64_t k_hi,
                                        int64_t *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        out[0] = static_cast<int64_t>(sorted[k_lo]);
        out[1] = static_cast<int64_t>(sorted[k_hi]);
        out[2] = static_cast<int64_t>(sorted[n - 1]);
    }
}

// out[0] = number of zero keys among the first n sorted 0/1 keys (= number of light rows)
__global__ void count_zero_keys_kernel(const uint64_t *__restrict__ sorted, int64_t n, int64_t *__restrict__ out) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int64_t lo = 0, hi = n;
        while (lo < hi) {
            const int64_t mid = lo + ((hi - lo) >> 1);
            if (sorted[mid] == 0)
                lo = mid + 1;
            else
                hi = mid;
        }
        out[0] = lo;
    }
}

}  // namespace gb
}  // namespace tgnn
