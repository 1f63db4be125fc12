// Runtime enum -> compile-time type dispatch used by the C-ABI entry points.
#pragma once

#include "launch.cuh"

namespace tgnn {

template <typename T>
struct TypeTag {
    using type = T;
};
template <int V>
struct IntTag {
    static constexpr int value = V;
};

// Calls f(TypeTag<T>, TypeTag<I>, IntTag<vpl>) for the runtime triple.
template <class F>
int32_t dispatch_tiv(int32_t dtype, int32_t itype, int vpl, F &&f) {
    auto with_v = [&](auto tt, auto it) -> int32_t {
        switch (vpl) {
            case 1: return f(tt, it, IntTag<1>{});
            case 2: return f(tt, it, IntTag<2>{});
            case 4: return f(tt, it, IntTag<4>{});
            case 8: return f(tt, it, IntTag<8>{});
            default: return fail(TGNN_ERR_UNSUPPORTED, "unsupported chunks per lane %d", vpl);
        }
    };
    auto with_i = [&](auto tt) -> int32_t {
        switch (itype) {
            case TGNN_I32: return with_v(tt, TypeTag<int32_t>{});
            case TGNN_I64: return with_v(tt, TypeTag<int64_t>{});
            default: return fail(TGNN_ERR_INVALID_ARGUMENT, "unknown index type %d", itype);
        }
    };
    switch (dtype) {
        case TGNN_F32: return with_i(TypeTag<float>{});
        case TGNN_F16: return with_i(TypeTag<__half>{});
        case TGNN_BF16: return with_i(TypeTag<__nv_bfloat16>{});
        default: return fail(TGNN_ERR_INVALID_ARGUMENT, "unknown element type %d", dtype);
    }
}

// Per-family scratch sizes (words of state per lane are op constants).
size_t reduce_scratch_bytes(int32_t op, int32_t dtype, int32_t itype, int64_t num_chunks, int64_t cols);
size_t gatv2_scratch_bytes(int32_t op, int32_t dtype, int32_t itype, int64_t num_chunks, int64_t cols);
size_t gt_scratch_bytes(int32_t op, int32_t dtype, int32_t itype, int64_t num_chunks, int64_t cols);

}  // namespace tgnn
