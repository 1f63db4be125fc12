// Per-row ops of the fused GATv2 aggregation: forward, destination-side
// backward (forward CSR) and source-side backward (transposed CSR).
//
//   z_ij = l_i + r_j          e_ij = sum_d a_d * LReLU(z_ijd)
//   alpha_ij = softmax_j(e_ij)        out_i = sum_j alpha_ij r_j
//   ge_ij = alpha_ij (<gh_i, r_j> - G_i),  G_i = <gh_i, out_i>
//   grad_l_i = sum_j ge_ij LReLU'(z_ij) * a        grad_a += ge_ij LReLU(z_ij)
//   grad_r_j = sum_i alpha_ij gh_i + ge_ij LReLU'(z_ij) * a
// LReLU'(z) is 1 for z > 0 and the negative slope otherwise.
#pragma once

#include "ops_attn.cuh"

namespace tgnn {

template <typename T>
struct Gatv2Params {
    const T *l;
    int64_t ldl;
    const T *r;
    int64_t ldr;
    const T *attn;  // [H, D]
    const T *gh;    // grad_out (backward only)
    int64_t ldg;
    const float *lse;  // [rows, H]
    const float *G;    // [rows, H]
    T *out;            // out (forward) | grad_l (bwd dst) | grad_r (bwd src)
    int64_t ldo;
    float *lse_out;      // forward
    float *grad_attn;    // bwd dst, fp32 [H, D]
    int cols;
    int heads;
    int head_dim;
    float slope;
};

// LReLU(z) = z + (slope - 1) * min(z, 0): two instructions, no select.
__device__ __forceinline__ float lrelu(float z, float slope_m1) { return fmaf(fminf(z, 0.0f), slope_m1, z); }

// Everything the three ops share: lane geometry, attention vector, slope.
template <typename T, typename I, int kVpl>
struct Gatv2Base {
    using index_t = I;
    using Params = Gatv2Params<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap hm;
    uint64_t keep;
    float slope_m1;
    float a[kVals];

    __device__ __forceinline__ Gatv2Base(const Params &p_, const Lanes &L_, float a_scale)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()),
          slope_m1(p_.slope - 1.0f) {
        load_span_f32<T, kVpl>(p.attn, map.off, a);
#pragma unroll
        for (int i = 0; i < kVals; ++i) a[i] *= a_scale;
    }
};

// ---- forward ----------------------------------------------------------------------
template <typename T, typename I, int kVpl>
struct Gatv2FwdOp : Gatv2Base<T, I, kVpl> {
    using B = Gatv2Base<T, I, kVpl>;
    using typename B::index_t;
    using typename B::Params;
    using B::a; using B::hm; using B::keep; using B::kVals; using B::L; using B::map; using B::p; using B::slope_m1;
    using Acc = SoftmaxAcc<kVals>;
    static constexpr int kWords = Acc::kWords;
    static constexpr int kUnroll = kVpl >= 4 ? 2 : 4;
    static constexpr int kCarryWords = 0;
    static constexpr int kLightMinBlocks = TGNN_MIN_BLOCKS_GATV2(kVpl);
    static constexpr int kLightMaxThreads = TGNN_ATTN_LIGHT_THREADS;

    struct Row {
        float l[kVals];
    };
    using State = Acc;
    using Carry = NoCarry;
    struct Frag {
        Span<kVpl> r;
    };

    // The attention vector is pre-multiplied by log2(e): scores come out in the base-2 domain.
    __device__ __forceinline__ Gatv2FwdOp(const Params &p_, const Lanes &L_) : B(p_, L_, kLog2e) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_span_f32<T, kVpl>(p.l + static_cast<int64_t>(row) * p.ldl, map.off, rc.l);
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_span<T, kVpl>(p.r + static_cast<int64_t>(src) * p.ldr, map.off, keep, f.r);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float sc[kUnroll];
        float x[kUnroll][kVals];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) f[u].r.clear();
            f[u].r.template to_f32<T>(x[u]);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < kVals; ++i) acc = fmaf(a[i], lrelu(rc.l[i] + x[u][i], slope_m1), acc);
            sc[u] = acc;
        }
        hm.finish(sc);
        if (!kAll) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u)
                if (!ok[u]) sc[u] = -INFINITY;
        }
        s.template push<kUnroll, kAll>(sc, x);
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0 || !map.live) return;
        const float inv = s.s > 0.0f ? 1.0f / s.s : 0.0f;
        float x[kVals];
#pragma unroll
        for (int i = 0; i < kVals; ++i) x[i] = s.acc[i] * inv;
        store_span_f32<T, kVpl>(p.out + static_cast<int64_t>(row) * p.ldo, map.off, x);
        if (hm.writer) p.lse_out[static_cast<int64_t>(row) * p.heads + hm.head] = s.lse();
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

// ---- backward, destination side (forward CSR) ------------------------------------------
template <typename T, typename I, int kVpl>
struct Gatv2BwdDstOp : Gatv2Base<T, I, kVpl> {
    using B = Gatv2Base<T, I, kVpl>;
    using typename B::index_t;
    using typename B::Params;
    using B::a; using B::hm; using B::keep; using B::kVals; using B::L; using B::map; using B::p; using B::slope_m1;
    static constexpr int kWords = 2 * kVals;  // grad_l | grad_a
    static constexpr int kUnroll = TGNN_ATTN_UNROLL(kVpl);
    static constexpr int kCarryWords = kVals;
    static constexpr int kLightMinBlocks = TGNN_MIN_BLOCKS_GATV2(kVpl);
    static constexpr int kLightMaxThreads = TGNN_ATTN_LIGHT_THREADS;

    struct Row {
        float l[kVals];
        float gh[kVals];
        float lse2;  // log-sum-exp in the base-2 domain
        float G;
    };
    using State = SumAcc<2 * kVals>;
    struct Carry {
        float ga[kVals];
    };
    struct Frag {
        Span<kVpl> r;
    };

    __device__ __forceinline__ Gatv2BwdDstOp(const Params &p_, const Lanes &L_) : B(p_, L_, 1.0f) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_span_f32<T, kVpl>(p.l + static_cast<int64_t>(row) * p.ldl, map.off, rc.l);
        load_span_f32<T, kVpl>(p.gh + static_cast<int64_t>(row) * p.ldg, map.off, rc.gh);
        const int64_t at = static_cast<int64_t>(row) * p.heads + hm.head;
        rc.lse2 = __ldg(p.lse + at) * kLog2e;
        rc.G = __ldg(p.G + at);
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_span<T, kVpl>(p.r + static_cast<int64_t>(src) * p.ldr, map.off, keep, f.r);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll];  // [edge score | <gh, r>] partial dot products
        float x[kUnroll][kVals];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) f[u].r.clear();
            f[u].r.template to_f32<T>(x[u]);
            float pe = 0.0f, pp = 0.0f;
#pragma unroll
            for (int i = 0; i < kVals; ++i) {
                pe = fmaf(a[i], lrelu(rc.l[i] + x[u][i], slope_m1), pe);
                pp = fmaf(rc.gh[i], x[u][i], pp);
            }
            d[u] = pe;
            d[kUnroll + u] = pp;
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float alpha = fast_exp2(fmaf(d[u], kLog2e, -rc.lse2));
            if (!kAll && !ok[u]) alpha = 0.0f;
            const float ge = alpha * (d[kUnroll + u] - rc.G);
            const float ge_neg = ge * p.slope;
#pragma unroll
            for (int i = 0; i < kVals; ++i) {
                const float z = rc.l[i] + x[u][i];
                s.a[i] = fmaf(z > 0.0f ? ge : ge_neg, a[i], s.a[i]);
                s.a[kVals + i] = fmaf(ge, lrelu(z, slope_m1), s.a[kVals + i]);
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0 || !map.live) return;
        store_span_f32<T, kVpl>(p.out + static_cast<int64_t>(row) * p.ldo, map.off, s.a);
    }
    // Heavy / hub rows: the row's grad_a goes straight to global memory.
    __device__ __forceinline__ void flush_row(State &s) {
        if (L.grp != 0 || !map.live) return;
#pragma unroll
        for (int i = 0; i < kVals; ++i) atomicAdd(p.grad_attn + map.off + i, s.a[kVals + i]);
    }
    // Light rows: grad_a rides in registers across the warp's rows, is summed over
    // the CTA in shared memory and leaves with one atomic per feature per CTA.
    __device__ __forceinline__ void carry_init(Carry &c) {
#pragma unroll
        for (int i = 0; i < kVals; ++i) c.ga[i] = 0.0f;
    }
    __device__ __forceinline__ void carry_add(Carry &c, const State &s) {
#pragma unroll
        for (int i = 0; i < kVals; ++i) c.ga[i] += s.a[kVals + i];
    }
    __device__ __forceinline__ void carry_flush(Carry &c, uint32_t *smem) {
        float *buf = reinterpret_cast<float *>(smem);
        const int warps = blockDim.x >> 5;
        const int warp = threadIdx.x >> 5;
#pragma unroll
        for (int i = 0; i < kVals; ++i) buf[(warp * kVals + i) * 32 + L.lane] = c.ga[i];
        __syncthreads();
        if (warp != 0 || L.grp != 0 || !map.live) return;
#pragma unroll
        for (int i = 0; i < kVals; ++i) {
            float tot = 0.0f;
            for (int w = 0; w < warps; ++w) tot += buf[(w * kVals + i) * 32 + L.lane];
            atomicAdd(p.grad_attn + map.off + i, tot);
        }
    }
};

// ---- backward, source side (transposed CSR: row = source j, column = destination i) -------
template <typename T, typename I, int kVpl>
struct Gatv2BwdSrcOp : Gatv2Base<T, I, kVpl> {
    using B = Gatv2Base<T, I, kVpl>;
    using typename B::index_t;
    using typename B::Params;
    using B::a; using B::hm; using B::keep; using B::kVals; using B::L; using B::map; using B::p; using B::slope_m1;
    static constexpr int kWords = kVals;
    static constexpr int kUnroll = TGNN_ATTN_UNROLL(kVpl);
    static constexpr int kCarryWords = 0;
    static constexpr int kLightMinBlocks = TGNN_MIN_BLOCKS_GATV2(kVpl);
    static constexpr int kLightMaxThreads = TGNN_ATTN_LIGHT_THREADS;

    struct Row {
        float r[kVals];
    };
    using State = SumAcc<kVals>;
    using Carry = NoCarry;
    struct Frag {
        Span<kVpl> l;
        Span<kVpl> g;
        float lse;
        float G;
    };

    __device__ __forceinline__ Gatv2BwdSrcOp(const Params &p_, const Lanes &L_) : B(p_, L_, 1.0f) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_span_f32<T, kVpl>(p.r + static_cast<int64_t>(row) * p.ldr, map.off, rc.r);
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I dst, Frag &f) {
        gather_span<T, kVpl>(p.l + static_cast<int64_t>(dst) * p.ldl, map.off, keep, f.l);
        gather_span<T, kVpl>(p.gh + static_cast<int64_t>(dst) * p.ldg, map.off, keep, f.g);
        const int64_t at = static_cast<int64_t>(dst) * p.heads + hm.head;
        f.lse = __ldg(p.lse + at);
        f.G = __ldg(p.G + at);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll];
        float xl[kUnroll][kVals], xg[kUnroll][kVals];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) {
                f[u].l.clear();
                f[u].g.clear();
                f[u].lse = f[u].G = 0.0f;
            }
            f[u].l.template to_f32<T>(xl[u]);
            f[u].g.template to_f32<T>(xg[u]);
            float pe = 0.0f, pp = 0.0f;
#pragma unroll
            for (int i = 0; i < kVals; ++i) {
                pe = fmaf(a[i], lrelu(xl[u][i] + rc.r[i], slope_m1), pe);
                pp = fmaf(xg[u][i], rc.r[i], pp);
            }
            d[u] = pe;
            d[kUnroll + u] = pp;
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float alpha = fast_exp2((d[u] - f[u].lse) * kLog2e);
            if (!kAll && !ok[u]) alpha = 0.0f;
            const float ge = alpha * (d[kUnroll + u] - f[u].G);
            const float ge_neg = ge * p.slope;
#pragma unroll
            for (int i = 0; i < kVals; ++i) {
                const float z = xl[u][i] + rc.r[i];
                s.a[i] = fmaf(alpha, xg[u][i], fmaf(z > 0.0f ? ge : ge_neg, a[i], s.a[i]));
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0 || !map.live) return;
        store_span_f32<T, kVpl>(p.out + static_cast<int64_t>(row) * p.ldo, map.off, s.a);
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

}  // namespace tgnn
