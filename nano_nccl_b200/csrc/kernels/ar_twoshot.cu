#include "kernels/dispatch.cuh"

#include <type_traits>

namespace nano_nccl::dev {

cudaError_t launch_ar_twoshot(const CommDev& c, const void* src, void* dst, std::size_t count,
                              DType dtype, RedOp op, bool multicast, const Geometry& g,
                              cudaStream_t stream) {
    return dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            if (multicast) {
                ar_twoshot_kernel<T, Op, true><<<g.grid, kCollectiveThreads, 0, stream>>>(
                    c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
            } else {
                ar_twoshot_kernel<T, Op, false><<<g.grid, kCollectiveThreads, 0, stream>>>(
                    c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
            }
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_ar_symm_p2p(const CommDev& c, const void* const* src_peers, void* const* dst_peers,
                               std::size_t bytes, DType dtype, RedOp op, bool one_shot, int grid,
                               cudaStream_t stream) {
    if (bytes % 16 != 0) return cudaErrorInvalidValue;
    SymmPeers p{};
    for (int r = 0; r < c.nranks; ++r) {
        p.src[r] = static_cast<const char*>(src_peers[r]);
        p.dst[r] = static_cast<char*>(dst_peers[r]);
    }
    const std::size_t nvec = bytes / 16;
    return dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            auto launch = [&](auto n_tag) {
                constexpr int kN = decltype(n_tag)::value;
                if (one_shot) {
                    ar_symm_p2p_kernel<T, Op, true, kN><<<grid, kCollectiveThreads, 0, stream>>>(c, p, nvec);
                } else {
                    ar_symm_p2p_kernel<T, Op, false, kN><<<grid, kCollectiveThreads, 0, stream>>>(c, p, nvec);
                }
            };
            switch (c.nranks) {  // the common rank counts get loops unrolled over the ranks with several vectors in flight
                case 2: launch(std::integral_constant<int, 2>{}); break;
                case 4: launch(std::integral_constant<int, 4>{}); break;
                case 8: launch(std::integral_constant<int, 8>{}); break;
                default: launch(std::integral_constant<int, 0>{}); break;
            }
            return cudaGetLastError();
        });
    });
}

}  // namespace nano_nccl::dev
