// Per-row ops of the fused graph-transformer attention: forward, destination-side
// backward (forward CSR, gives dK) and source-side backward (transposed CSR,
// gives dQ and dV).  Destination i, source j:
//
//   s_ij = scale <q_j, k_i>      alpha_ij = softmax_j(s_ij)     out_i = sum_j alpha_ij v_j
//   dS_ij = alpha_ij (<dO_i, v_j> - Delta_i),  Delta_i = <dO_i, out_i>
//   dk_i = sum_j scale dS_ij q_j     dq_j = sum_i scale dS_ij k_i     dv_j = sum_i alpha_ij dO_i
//
// Both backward halves recompute alpha from the saved log-sum-exp; neither uses atomics.
#pragma once

#include "ops_attn.cuh"

namespace tgnn {

template <typename T>
struct GtParams {
    const T *q;
    int64_t ldq;
    const T *k;
    int64_t ldk;
    const T *v;
    int64_t ldv;
    const T *d_out;
    int64_t ldd;
    const float *lse;
    const float *delta;
    T *out0;  // out (forward) | dk (bwd dst) | dq (bwd src)
    int64_t ldo0;
    T *out1;  // dv (bwd src)
    int64_t ldo1;
    float *lse_out;
    int cols;
    int heads;
    int head_dim;
    float scale;
};

template <int kVpl>
__device__ __forceinline__ void clear_chunks(uint4 (&raw)[kVpl]) {
#pragma unroll
    for (int v = 0; v < kVpl; ++v) raw[v] = make_uint4(0u, 0u, 0u, 0u);
}

// ---- forward ----------------------------------------------------------------------
template <typename T, typename I, int kVpl>
struct GtFwdOp {
    using index_t = I;
    using Params = GtParams<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    using Acc = SoftmaxAcc<kVpl, kPer>;
    static constexpr int kWords = Acc::kWords;
    static constexpr int kUnroll = kVpl >= 4 ? 1 : 2;
    static constexpr int kCarryWords = 0;

    struct Row {
        float k[kVals];  // key row times scale * log2(e)
    };
    using State = Acc;
    using Carry = NoCarry;
    struct Frag {
        uint4 rawq[kVpl];
        uint4 rawv[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;

    __device__ __forceinline__ GtFwdOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.k + static_cast<int64_t>(row) * p.ldk, map, rc.k);
        const float f = p.scale * kLog2e;
#pragma unroll
        for (int i = 0; i < kVals; ++i) rc.k[i] *= f;
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_row<T, kVpl>(p.q + static_cast<int64_t>(src) * p.ldq, map, keep, f.rawq);
        gather_row<T, kVpl>(p.v + static_cast<int64_t>(src) * p.ldv, map, keep, f.rawv);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float sc[kUnroll * kVpl];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) {
                clear_chunks<kVpl>(f[u].rawq);
                clear_chunks<kVpl>(f[u].rawv);
            }
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float x[kPer];
                Elem<T>::unpack(f[u].rawq[v], x);
                float acc = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) acc = fmaf(x[e], rc.k[v * kPer + e], acc);
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
                Elem<T>::unpack(f[u].rawv[v], x[u]);
            }
            s.template push<kUnroll, kAll>(v, s2, x);
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        T *orow = p.out0 + static_cast<int64_t>(row) * p.ldo0;
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

// ---- backward, destination side: dk over the forward CSR ----------------------------------
template <typename T, typename I, int kVpl>
struct GtBwdDstOp {
    using index_t = I;
    using Params = GtParams<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = kVals;
    static constexpr int kUnroll = kVpl >= 4 ? 1 : 2;
    static constexpr int kCarryWords = 0;

    struct Row {
        float k[kVals];  // times scale * log2(e)
        float dO[kVals];
        float lse2[kVpl];
        float delta[kVpl];
    };
    using State = SumAcc<kVals>;
    using Carry = NoCarry;
    struct Frag {
        uint4 rawq[kVpl];
        uint4 rawv[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;

    __device__ __forceinline__ GtBwdDstOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.k + static_cast<int64_t>(row) * p.ldk, map, rc.k);
        load_row_f32<T, kVpl>(p.d_out + static_cast<int64_t>(row) * p.ldd, map, rc.dO);
        const float f = p.scale * kLog2e;
#pragma unroll
        for (int i = 0; i < kVals; ++i) rc.k[i] *= f;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const int64_t at = static_cast<int64_t>(row) * p.heads + hm.head[v];
            rc.lse2[v] = __ldg(p.lse + at) * kLog2e;
            rc.delta[v] = __ldg(p.delta + at);
        }
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I src, Frag &f) {
        gather_row<T, kVpl>(p.q + static_cast<int64_t>(src) * p.ldq, map, keep, f.rawq);
        gather_row<T, kVpl>(p.v + static_cast<int64_t>(src) * p.ldv, map, keep, f.rawv);
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll * kVpl];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) {
                clear_chunks<kVpl>(f[u].rawq);
                clear_chunks<kVpl>(f[u].rawv);
            }
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float xq[kPer], xv[kPer];
                Elem<T>::unpack(f[u].rawq[v], xq);
                Elem<T>::unpack(f[u].rawv[v], xv);
                float ps = 0.0f, pd = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    ps = fmaf(xq[e], rc.k[v * kPer + e], ps);
                    pd = fmaf(xv[e], rc.dO[v * kPer + e], pd);
                }
                d[u * kVpl + v] = ps;
                d[(kUnroll + u) * kVpl + v] = pd;
            }
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float alpha = fast_exp2(d[u * kVpl + v] - rc.lse2[v]);
                if (!kAll && !ok[u]) alpha = 0.0f;
                const float ds = alpha * (d[(kUnroll + u) * kVpl + v] - rc.delta[v]) * p.scale;
                float xq[kPer];
                Elem<T>::unpack(f[u].rawq[v], xq);
#pragma unroll
                for (int e = 0; e < kPer; ++e) s.a[v * kPer + e] = fmaf(ds, xq[e], s.a[v * kPer + e]);
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        store_row_f32<T, kVpl>(p.out0 + static_cast<int64_t>(row) * p.ldo0, map, s.a);
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

// ---- backward, source side: dq and dv over the transposed CSR --------------------------------
template <typename T, typename I, int kVpl>
struct GtBwdSrcOp {
    using index_t = I;
    using Params = GtParams<T>;
    static constexpr int kPer = Elem<T>::kPerChunk;
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = 2 * kVals;  // dq | dv
    static constexpr int kUnroll = kVpl >= 4 ? 1 : 2;
    static constexpr int kCarryWords = 0;

    struct Row {
        float q[kVals];  // times scale * log2(e)
        float v[kVals];
    };
    using State = SumAcc<2 * kVals>;
    using Carry = NoCarry;
    struct Frag {
        uint4 rawk[kVpl];
        uint4 rawd[kVpl];
        float lse[kVpl];
        float delta[kVpl];
    };

    const Params &p;
    const Lanes &L;
    AttnMap<kVpl, kPer> map;
    HeadMap<kVpl, kPer> hm;
    uint64_t keep;

    __device__ __forceinline__ GtBwdSrcOp(const Params &p_, const Lanes &L_)
        : p(p_), L(L_), map(L_, p_.cols), hm(L_, map, p_.head_dim), keep(make_keep_policy()) {}
    __device__ __forceinline__ void row_begin(I row, Row &rc) {
        load_row_f32<T, kVpl>(p.q + static_cast<int64_t>(row) * p.ldq, map, rc.q);
        load_row_f32<T, kVpl>(p.v + static_cast<int64_t>(row) * p.ldv, map, rc.v);
        const float f = p.scale * kLog2e;
#pragma unroll
        for (int i = 0; i < kVals; ++i) rc.q[i] *= f;
    }
    __device__ __forceinline__ void init(State &s) { s.init(); }
    __device__ __forceinline__ void load(I dst, Frag &f) {
        gather_row<T, kVpl>(p.k + static_cast<int64_t>(dst) * p.ldk, map, keep, f.rawk);
        gather_row<T, kVpl>(p.d_out + static_cast<int64_t>(dst) * p.ldd, map, keep, f.rawd);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const int64_t at = static_cast<int64_t>(dst) * p.heads + hm.head[v];
            f.lse[v] = __ldg(p.lse + at);
            f.delta[v] = __ldg(p.delta + at);
        }
    }
    template <bool kAll>
    __device__ __forceinline__ void consume(const Row &rc, State &s, Frag (&f)[kUnroll], const I (&)[kUnroll],
                                            const I (&)[kUnroll], const bool (&ok)[kUnroll]) {
        float d[2 * kUnroll * kVpl];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!kAll && !ok[u]) {
                clear_chunks<kVpl>(f[u].rawk);
                clear_chunks<kVpl>(f[u].rawd);
#pragma unroll
                for (int v = 0; v < kVpl; ++v) f[u].lse[v] = f[u].delta[v] = 0.0f;
            }
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float xk[kPer], xd[kPer];
                Elem<T>::unpack(f[u].rawk[v], xk);
                Elem<T>::unpack(f[u].rawd[v], xd);
                float ps = 0.0f, pd = 0.0f;
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    ps = fmaf(xk[e], rc.q[v * kPer + e], ps);
                    pd = fmaf(xd[e], rc.v[v * kPer + e], pd);
                }
                d[u * kVpl + v] = ps;
                d[(kUnroll + u) * kVpl + v] = pd;
            }
        }
        hm.finish(d);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                float alpha = fast_exp2(fmaf(-f[u].lse[v], kLog2e, d[u * kVpl + v]));
                if (!kAll && !ok[u]) alpha = 0.0f;
                const float ds = alpha * (d[(kUnroll + u) * kVpl + v] - f[u].delta[v]) * p.scale;
                float xk[kPer], xd[kPer];
                Elem<T>::unpack(f[u].rawk[v], xk);
                Elem<T>::unpack(f[u].rawd[v], xd);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const int i = v * kPer + e;
                    s.a[i] = fmaf(ds, xk[e], s.a[i]);
                    s.a[kVals + i] = fmaf(alpha, xd[e], s.a[kVals + i]);
                }
            }
        }
    }
    __device__ __forceinline__ void merge(State &s, const State &o) { s.merge(o); }
    __device__ __forceinline__ void to_words(const State &s, uint32_t *w) { s.to_words(w); }
    __device__ __forceinline__ void from_words(State &s, const uint32_t *w) { s.from_words(w); }
    __device__ __forceinline__ void row_end(I row, const Row &, State &s, I) {
        if (L.grp != 0) return;
        store_row_f32<T, kVpl>(p.out0 + static_cast<int64_t>(row) * p.ldo0, map, s.a);
        store_row_f32<T, kVpl>(p.out1 + static_cast<int64_t>(row) * p.ldo1, map, s.a + kVals);
    }
    __device__ __forceinline__ void flush_row(State &) {}
    __device__ __forceinline__ void carry_init(Carry &) {}
    __device__ __forceinline__ void carry_add(Carry &, const State &) {}
    __device__ __forceinline__ void carry_flush(Carry &, uint32_t *) {}
};

}  // namespace tgnn
