// Shared pieces of the fused attention ops (GATv2 and graph transformer).
//
// A node row is [heads * head_dim]; a warp (or a group of G lanes) covers it in
// 16-byte chunks, lane-contiguous, so one head occupies `lanes_per_head`
// consecutive lanes of one chunk index v (or, for head_dim > 32 chunks, all 32
// lanes of several v).  Per-head dot products are finished with xor shuffles
// inside that lane range; every lane of a head then holds the head's score and
// runs the softmax bookkeeping for its own accumulators redundantly.
//
// Edges are folded in batches of kUnroll: all scores of a batch are reduced by
// one unrolled shuffle tree, the running maximum moves once per batch, and the
// accumulators are rescaled once per batch.  Softmax runs in the base-2 domain
// (scores are pre-multiplied by log2 e, `ex2.approx` / `lg2.approx`).
#pragma once

#include "ops_reduce.cuh"

namespace tgnn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Chunk offsets for the attention ops: chunks beyond the row are clamped to
// offset 0 so that the edge loop needs no per-chunk predicate (their lanes
// compute values nobody stores; a head never mixes clamped and real chunks
// because rows end on a head boundary).  `live[v]` gates the stores.
template <int kVpl, int kPer>
struct AttnMap {
    int off[kVpl];
    bool live[kVpl];
    __device__ __forceinline__ AttnMap(const Lanes &L, int cols) {
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const int o = ((L.slice * kVpl + v) * L.G + L.g_lane) * kPer;
            live[v] = o < cols;
            off[v] = live[v] ? o : 0;
        }
    }
};

// Head layout of one lane.
template <int kVpl, int kPer>
struct HeadMap {
    int lanes_per_head;  // shuffle span, <= 32
    int v_per_head;      // chunk indices v that belong to one head (1 unless head_dim > 32 chunks)
    int head[kVpl];      // head index of chunk v
    bool writer[kVpl];   // this lane stores the per-head scalars of chunk v's head

    __device__ __forceinline__ HeadMap(const Lanes &L, const AttnMap<kVpl, kPer> &map, int head_dim) {
        const int cph = head_dim / kPer;
        lanes_per_head = cph > 32 ? 32 : cph;
        v_per_head = cph > 32 ? cph / 32 : 1;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            head[v] = map.off[v] / head_dim;
            writer[v] = map.live[v] && (map.off[v] % head_dim) == 0 && L.grp == 0;
        }
    }

    template <int kLanes, int kN>
    __device__ __forceinline__ static void tree(float (&x)[kN]) {
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) {
#pragma unroll
            for (int i = 0; i < kN; ++i) x[i] += __shfl_xor_sync(kFull, x[i], o);
        }
    }

    // x[j * kVpl + v]: this lane's partial dot product over chunk v (j = edge of
    // the batch, or any other outer index).  On return every entry is the full
    // dot product of its head, in every lane of that head.
    template <int kN>
    __device__ __forceinline__ void finish(float (&x)[kN]) const {
        if (v_per_head > 1) {
#pragma unroll
            for (int j = 0; j < kN / kVpl; ++j) {
                float tot[kVpl];
#pragma unroll
                for (int v = 0; v < kVpl; ++v) {
                    tot[v] = 0.0f;
#pragma unroll
                    for (int u = 0; u < kVpl; ++u)
                        if (u / v_per_head == v / v_per_head) tot[v] += x[j * kVpl + u];
                }
#pragma unroll
                for (int v = 0; v < kVpl; ++v) x[j * kVpl + v] = tot[v];
            }
        }
        switch (lanes_per_head) {  // warp-uniform
            case 32: tree<32>(x); break;
            case 16: tree<16>(x); break;
            case 8: tree<8>(x); break;
            case 4: tree<4>(x); break;
            case 2: tree<2>(x); break;
            default: break;
        }
    }
};

// Running softmax-weighted sum of gathered rows (base-2 domain): per chunk v a
// running max m, a running denominator s and kPer numerators.
template <int kVpl, int kPer>
struct SoftmaxAcc {
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = kVals + 2 * kVpl;
    float acc[kVals];
    float m[kVpl];
    float s[kVpl];

    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < kVals; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            m[v] = -INFINITY;
            s[v] = 0.0f;
        }
    }
    // Fold a batch of kU edges into chunk v.  sc[j]: base-2 score of edge j for
    // chunk v's head (-inf for an absent edge when !kAll); x[j]: the value chunk.
    // Returns nothing; with !kAll a batch without any edge leaves the state as is.
    template <int kU, bool kAll>
    __device__ __forceinline__ void push(int v, const float (&sc)[kU], const float (&x)[kU][kPer]) {
        float m_new = m[v];
#pragma unroll
        for (int j = 0; j < kU; ++j) m_new = fmaxf(m_new, sc[j]);
        if (!kAll && m_new == -INFINITY) return;
        const float corr = fast_exp2(m[v] - m_new);  // 0 for the first batch (m = -inf)
        float p[kU];
        float psum = 0.0f;
#pragma unroll
        for (int j = 0; j < kU; ++j) {
            p[j] = fast_exp2(sc[j] - m_new);
            psum += p[j];
        }
        s[v] = fmaf(s[v], corr, psum);
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            float a = acc[v * kPer + e] * corr;
#pragma unroll
            for (int j = 0; j < kU; ++j) a = fmaf(p[j], x[j][e], a);
            acc[v * kPer + e] = a;
        }
        m[v] = m_new;
    }
    __device__ __forceinline__ void merge(const SoftmaxAcc &o) {
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const float m_new = fmaxf(m[v], o.m[v]);
            const float c1 = m[v] == -INFINITY ? 0.0f : fast_exp2(m[v] - m_new);
            const float c2 = o.m[v] == -INFINITY ? 0.0f : fast_exp2(o.m[v] - m_new);
            s[v] = s[v] * c1 + o.s[v] * c2;
#pragma unroll
            for (int e = 0; e < kPer; ++e) acc[v * kPer + e] = acc[v * kPer + e] * c1 + o.acc[v * kPer + e] * c2;
            m[v] = m_new;
        }
    }
    // Natural-log log-sum-exp of chunk v's head; -inf for a row without edges.
    __device__ __forceinline__ float lse(int v) const {
        return s[v] > 0.0f ? (m[v] + fast_log2(s[v])) * kLn2 : -INFINITY;
    }
    __device__ __forceinline__ void to_words(uint32_t *w) const {
#pragma unroll
        for (int i = 0; i < kVals; ++i) w[i] = __float_as_uint(acc[i]);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            w[kVals + v] = __float_as_uint(m[v]);
            w[kVals + kVpl + v] = __float_as_uint(s[v]);
        }
    }
    __device__ __forceinline__ void from_words(const uint32_t *w) {
#pragma unroll
        for (int i = 0; i < kVals; ++i) acc[i] = __uint_as_float(w[i]);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            m[v] = __uint_as_float(w[kVals + v]);
            s[v] = __uint_as_float(w[kVals + kVpl + v]);
        }
    }
};

// Plain per-lane float accumulators (the backward ops).
template <int kN>
struct SumAcc {
    float a[kN];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] = 0.0f;
    }
    __device__ __forceinline__ void merge(const SumAcc &o) {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] += o.a[i];
    }
    __device__ __forceinline__ void to_words(uint32_t *w) const {
#pragma unroll
        for (int i = 0; i < kN; ++i) w[i] = __float_as_uint(a[i]);
    }
    __device__ __forceinline__ void from_words(const uint32_t *w) {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] = __uint_as_float(w[i]);
    }
};

// Row-local operand: the chunks of one row as floats (clamped chunks read offset 0).
template <typename T, int kVpl>
__device__ __forceinline__ void load_row_f32(const T *row, const AttnMap<kVpl, Elem<T>::kPerChunk> &map, float *dst) {
    constexpr int kPer = Elem<T>::kPerChunk;
#pragma unroll
    for (int v = 0; v < kVpl; ++v) Elem<T>::unpack(ld_stream16(row + map.off[v]), dst + v * kPer);
}

template <typename T, int kVpl>
__device__ __forceinline__ void store_row_f32(T *row, const AttnMap<kVpl, Elem<T>::kPerChunk> &map, const float *src) {
    constexpr int kPer = Elem<T>::kPerChunk;
#pragma unroll
    for (int v = 0; v < kVpl; ++v)
        if (map.live[v]) st_stream16(row + map.off[v], Elem<T>::pack(src + v * kPer));
}

template <typename T, int kVpl>
__device__ __forceinline__ void gather_row(const T *row, const AttnMap<kVpl, Elem<T>::kPerChunk> &map, uint64_t keep,
                                           uint4 *raw) {
#pragma unroll
    for (int v = 0; v < kVpl; ++v) raw[v] = ld_gather16(row + map.off[v], keep);
}

// Empty hooks for ops that carry nothing across rows.
struct NoCarry {};

}  // namespace tgnn
