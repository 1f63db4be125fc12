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

template <int kVpl>
__device__ __forceinline__ void clear_frag(uint4 (&raw)[kVpl]) {
#pragma unroll
    for (int v = 0; v < kVpl; ++v) raw[v] = make_uint4(0u, 0u, 0u, 0u);
}

// ---- forward ----------------------------------------------------------------------
template <typename T, typename I, int kVpl>
struct Gatv2FwdOp {
    using index_t = I;
    using Params = Gatv2Params<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    using Acc = SoftmaxAcc<kVpl, kPer>;
    static constexpr int kWords = Acc::kWords;
    static constexpr int kUnroll = kVpl >= 4 ? 2 : 4;
    static constexpr int kCarryWords = 0;

    struct Row {
        float l[kVals];
    };
    using State = Acc;
    using Carry = NoCarry;
    struct Frag {
        uint4 raw[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;
    float slope_m1;
    float a[kVals];  // attention vector times log2(e): scores come out in the base-2 domain

    __device__ __forceinline__ Gatv2FwdOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()),
          slope_m1(p_.slope - 1.0f) {
        load_row_f32<T, kVpl>(p.attn, map, a);
#pragma unroll
        for (int i = 0; i < kVals; ++i) a[i] *= kLog2e;
    }
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.l + static_cast<int64_t>(row) * p.ldl, map, rc.l);
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_row<T, kVpl>(p.r + static_cast<int64_t>(src) * p.ldr, map, keep, f.raw);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float sc[kUnroll * kVpl];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) clear_frag<kVpl>(f[u].raw);
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float x[kPer];
                Elem<T>::unpack(f[u].raw[v], x);
                float acc = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e)
                    acc = fmaf(a[v * kPer + e], lrelu(rc.l[v * kPer + e] + x[e], slope_m1), acc);
                sc[u * kVpl + v] = acc;
            }
        }
        hm.finish(sc);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            float s2[kUnroll];
            float x[kUnroll][kPer];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                s2[u] = (kAll || ok[u]) ? sc[u * kVpl + v] : -INFINITY;
                Elem<T>::unpack(f[u].raw[v], x[u]);
            }
            s.template push<kUnroll, kAll>(v, s2, x);
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        T *orow = p.out + static_cast<int64_t>(row) * p.ldo;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            if (!map.live[v]) continue;
            const float inv = s.s[v] > 0.0f ? 1.0f / s.s[v] : 0.0f;
            float x[kPer];
#pragma unroll
            for (int e = 0; e < kPer; ++e) x[e] = s.acc[v * kPer + e] * inv;
            st_stream16(orow + map.off[v], Elem<T>::pack(x));
            if (hm.writer[v]) p.lse_out[static_cast<int64_t>(row) * p.heads + hm.head[v]] = s.lse(v);
        }
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

// ---- backward, destination side (forward CSR) ------------------------------------------
template <typename T, typename I, int kVpl>
struct Gatv2BwdDstOp {
    using index_t = I;
    using Params = Gatv2Params<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = 2 * kVals;  // grad_l | grad_a
    static constexpr int kUnroll = kVpl >= 4 ? 1 : 2;
    static constexpr int kCarryWords = kVals;

    struct Row {
        float l[kVals];
        float gh[kVals];
        float lse2[kVpl];  // log-sum-exp in the base-2 domain
        float G[kVpl];
    };
    using State = SumAcc<2 * kVals>;
    struct Carry {
        float ga[kVals];
    };
    struct Frag {
        uint4 raw[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;
    float slope_m1;
    float a[kVals];

    __device__ __forceinline__ Gatv2BwdDstOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()),
          slope_m1(p_.slope - 1.0f) {
        load_row_f32<T, kVpl>(p.attn, map, a);
    }
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.l + static_cast<int64_t>(row) * p.ldl, map, rc.l);
        load_row_f32<T, kVpl>(p.gh + static_cast<int64_t>(row) * p.ldg, map, rc.gh);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const int64_t at = static_cast<int64_t>(row) * p.heads + hm.head[v];
            rc.lse2[v] = __ldg(p.lse + at) * kLog2e;
            rc.G[v] = __ldg(p.G + at);
        }
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_row<T, kVpl>(p.r + static_cast<int64_t>(src) * p.ldr, map, keep, f.raw);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll * kVpl];  // [edge score | <gh, r>] partial dot products
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) clear_frag<kVpl>(f[u].raw);
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float x[kPer];
                Elem<T>::unpack(f[u].raw[v], x);
                float pe = 0.0f, pp = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const int i = v * kPer + e;
                    pe = fmaf(a[i], lrelu(rc.l[i] + x[e], slope_m1), pe);
                    pp = fmaf(rc.gh[i], x[e], pp);
                }
                d[u * kVpl + v] = pe;
                d[(kUnroll + u) * kVpl + v] = pp;
            }
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float alpha = fast_exp2(fmaf(d[u * kVpl + v], kLog2e, -rc.lse2[v]));
                if (!kAll && !ok[u]) alpha = 0.0f;
                const float ge = alpha * (d[(kUnroll + u) * kVpl + v] - rc.G[v]);
                const float ge_neg = ge * p.slope;
                float x[kPer];
                Elem<T>::unpack(f[u].raw[v], x);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const int i = v * kPer + e;
                    const float z = rc.l[i] + x[e];
                    s.a[i] = fmaf(z > 0.0f ? ge : ge_neg, a[i], s.a[i]);
                    s.a[kVals + i] = fmaf(ge, lrelu(z, slope_m1), s.a[kVals + i]);
                }
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        store_row_f32<T, kVpl>(p.out + static_cast<int64_t>(row) * p.ldo, map, s.a);
    }
    // Heavy / hub rows: the row's grad_a goes straight to global memory.
    __device__ __forceinline__ void flush_row(State &s) {
        if (L.grp != 0) return;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            if (!map.live[v]) continue;
#pragma unroll
            for (int e = 0; e < kPer; ++e) atomicAdd(p.grad_attn + map.off[v] + e, s.a[kVals + v * kPer + e]);
        }
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
        if (warp != 0 || L.grp != 0) return;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            if (!map.live[v]) continue;
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                const int i = v * kPer + e;
                float tot = 0.0f;
                for (int w = 0; w < warps; ++w) tot += buf[(w * kVals + i) * 32 + L.lane];
                atomicAdd(p.grad_attn + map.off[v] + e, tot);
            }
        }
    }
};

// ---- backward, source side (transposed CSR: row = source j, column = destination i) -------
template <typename T, typename I, int kVpl>
struct Gatv2BwdSrcOp {
    using index_t = I;
    using Params = Gatv2Params<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = kVals;
    static constexpr int kUnroll = kVpl >= 4 ? 1 : 2;
    static constexpr int kCarryWords = 0;

    struct Row {
        float r[kVals];
    };
    using State = SumAcc<kVals>;
    using Carry = NoCarry;
    struct Frag {
        uint4 rawl[kVpl];
        uint4 rawg[kVpl];
        float lse[kVpl];
        float G[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;
    float slope_m1;
    float a[kVals];

    __device__ __forceinline__ Gatv2BwdSrcOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()),
          slope_m1(p_.slope - 1.0f) {
        load_row_f32<T, kVpl>(p.attn, map, a);
    }
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.r + static_cast<int64_t>(row) * p.ldr, map, rc.r);
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I dst, Frag &f) {
        gather_row<T, kVpl>(p.l + static_cast<int64_t>(dst) * p.ldl, map, keep, f.rawl);
        gather_row<T, kVpl>(p.gh + static_cast<int64_t>(dst) * p.ldg, map, keep, f.rawg);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const int64_t at = static_cast<int64_t>(dst) * p.heads + hm.head[v];
            f.lse[v] = __ldg(p.lse + at);
            f.G[v] = __ldg(p.G + at);
        }
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll * kVpl];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) {
                clear_frag<kVpl>(f[u].rawl);
                clear_frag<kVpl>(f[u].rawg);
#pragma unroll
                for (int v = 0; v < kVpl; ++v) f[u].lse[v] = f[u].G[v] = 0.0f;
            }
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float xl[kPer], xg[kPer];
                Elem<T>::unpack(f[u].rawl[v], xl);
                Elem<T>::unpack(f[u].rawg[v], xg);
                float pe = 0.0f, pp = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const int i = v * kPer + e;
                    pe = fmaf(a[i], lrelu(xl[e] + rc.r[i], slope_m1), pe);
                    pp = fmaf(xg[e], rc.r[i], pp);
                }
                d[u * kVpl + v] = pe;
                d[(kUnroll + u) * kVpl + v] = pp;
            }
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float alpha = fast_exp2((d[u * kVpl + v] - f[u].lse[v]) * kLog2e);
                if (!kAll && !ok[u]) alpha = 0.0f;
                const float ge = alpha * (d[(kUnroll + u) * kVpl + v] - f[u].G[v]);
                const float ge_neg = ge * p.slope;
                float xl[kPer], xg[kPer];
                Elem<T>::unpack(f[u].rawl[v], xl);
                Elem<T>::unpack(f[u].rawg[v], xg);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const int i = v * kPer + e;
                    const float z = xl[e] + rc.r[i];
                    s.a[i] = fmaf(alpha, xg[e], fmaf(z > 0.0f ? ge : ge_neg, a[i], s.a[i]));
                }
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        store_row_f32<T, kVpl>(p.out + static_cast<int64_t>(row) * p.ldo, map, s.a);
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

}  // namespace tgnn
