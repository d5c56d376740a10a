// xnor-popcount GEMM entry points: argument checks and the choice of
// instruction path (CUDA-core POPC, legacy b1 mma.sync, tcgen05 kind::i8).
#include "common.cuh"
#include "gemm_popc.cuh"
#include "gemm_mma_b1.cuh"
#include "gemm_tcgen05_pair.cuh"

#include <cstdlib>
#include <cstring>

namespace bb {

struct GemmArgs {
    const uint64_t* A; const uint64_t* B;
    int64_t M, N, Kp, K;
    // plain output
    int32_t* C; int64_t ldc;
    // fused scale + sign + pack output
    const float* scale; uint64_t* out; int mode;
    bool pack;
    int leave_sms = 0;          // SMs the persistent tensor-core kernel leaves to other streams
};

static int run_popc(const GemmArgs& g, cudaStream_t st) {
    const dim3 grid((unsigned)((g.N + PG_BN - 1) / PG_BN), (unsigned)((g.M + PG_BM - 1) / PG_BM));
    BB_REQUIRE(grid.y <= 65535, BRUTE_ERR_UNSUPPORTED);
    if (!g.pack) {
        EpilogueInt32 ep{g.C, g.ldc, g.M, g.N};
        k_xnor_gemm_popc<<<grid, PG_THREADS, 0, st>>>(g.A, g.B, g.M, g.N, g.Kp, (int32_t)g.K, ep);
    } else {
        EpilogueScaleSignPack ep{g.scale, g.out, (g.N + 63) / 64, g.M, g.N, g.mode};
        k_xnor_gemm_popc<<<grid, PG_THREADS, 0, st>>>(g.A, g.B, g.M, g.N, g.Kp, (int32_t)g.K, ep);
    }
    return launch_status();
}

static bool mma_b1_accepts(const GemmArgs& g) {
    return g.Kp > 0 && (g.Kp % 2) == 0 && aligned16(g.A) && aligned16(g.B) &&
           (g.M + MB_BM - 1) / MB_BM <= 65535;
}

static int run_mma_b1(const GemmArgs& g, cudaStream_t st) {
    BB_REQUIRE(mma_b1_accepts(g), BRUTE_ERR_UNSUPPORTED);
    const dim3 grid((unsigned)((g.N + MB_BN - 1) / MB_BN), (unsigned)((g.M + MB_BM - 1) / MB_BM));
    auto* A8 = reinterpret_cast<const uint8_t*>(g.A);
    auto* B8 = reinterpret_cast<const uint8_t*>(g.B);
    if (!g.pack) {
        if (!kernel_smem_ready<k_xnor_gemm_mma_b1<false>>(MB_SMEM)) return BRUTE_ERR_LAUNCH;
        k_xnor_gemm_mma_b1<false><<<grid, MB_THREADS, MB_SMEM, st>>>(
            A8, B8, g.M, g.N, g.Kp * 8, (int32_t)g.K, g.C, g.ldc, nullptr, nullptr, 0, 0);
    } else {
        if (!kernel_smem_ready<k_xnor_gemm_mma_b1<true>>(MB_SMEM)) return BRUTE_ERR_LAUNCH;
        k_xnor_gemm_mma_b1<true><<<grid, MB_THREADS, MB_SMEM, st>>>(
            A8, B8, g.M, g.N, g.Kp * 8, (int32_t)g.K, nullptr, 0, g.scale,
            reinterpret_cast<uint32_t*>(g.out), 2 * ((g.N + 63) / 64), g.mode);
    }
    return launch_status();
}

static int env_impl() {
    // BRUTE_GEMM_IMPL overrides AUTO so that profiler runs can compare the pipes.
    static int cached = -1;
    if (cached >= 0) return cached;
    const char* e = std::getenv("BRUTE_GEMM_IMPL");
    int v = BRUTE_GEMM_AUTO;
    if (e) {
        if (!std::strcmp(e, "popc")) v = BRUTE_GEMM_POPC;
        else if (!std::strcmp(e, "b1") || !std::strcmp(e, "mma_b1")) v = BRUTE_GEMM_MMA_B1;
        else if (!std::strcmp(e, "i8") || !std::strcmp(e, "tcgen05")) v = BRUTE_GEMM_TCGEN05;
        else if (!std::strcmp(e, "i8x2") || !std::strcmp(e, "tcgen05_pair")) v = BRUTE_GEMM_TCGEN05_PAIR;
    }
    cached = v;
    return v;
}

static int dispatch(const GemmArgs& g, int impl, cudaStream_t st) {
    if (impl == BRUTE_GEMM_AUTO) {
        // the environment override applies only where that path accepts the shape
        const int e = env_impl();
        if (e == BRUTE_GEMM_POPC) impl = e;
        else if (e == BRUTE_GEMM_MMA_B1 && mma_b1_accepts(g)) impl = e;
        else if (e == BRUTE_GEMM_TCGEN05 && tc5_accepts(g.A, g.B, g.M, g.N, g.Kp)) impl = e;
        else if (e == BRUTE_GEMM_TCGEN05_PAIR && tc5_accepts(g.A, g.B, g.M, g.N, g.Kp) && tc5_pair_accepts(g.M, g.N)) impl = e;
    }
    if (impl == BRUTE_GEMM_AUTO) {
        // The tcgen05 kernels take every shape their TMA maps can describe, down to one row: even
        // a single mostly empty tile (28 us for 1 x 4096 x 4096 from an eager call, of which
        // about 25 are the call itself) beats the serial K loops of the other two paths
        // (84 us CUDA cores, 190 us mma.sync b1 at K = 4096). The CUDA-core path has no shape
        // rules at all and takes the rest (odd word counts, unaligned operands).
        if (tc5_accepts(g.A, g.B, g.M, g.N, g.Kp))
            impl = tc5_pair_prefers(g.M, g.N) ? BRUTE_GEMM_TCGEN05_PAIR : BRUTE_GEMM_TCGEN05;
        else if (mma_b1_accepts(g) && g.M * g.N >= 64 * 64) impl = BRUTE_GEMM_MMA_B1;
        else impl = BRUTE_GEMM_POPC;
    }
    switch (impl) {
        case BRUTE_GEMM_POPC:   return run_popc(g, st);
        case BRUTE_GEMM_MMA_B1: return run_mma_b1(g, st);
        case BRUTE_GEMM_TCGEN05:
            return tc5_run(g.A, g.B, g.M, g.N, g.Kp, g.K, g.C, g.ldc, g.scale, g.out, g.mode, g.pack, st);
        case BRUTE_GEMM_TCGEN05_PAIR:
            return tc5_pair_run(g.A, g.B, g.M, g.N, g.Kp, g.K, g.C, g.ldc, g.scale, g.out, g.mode, g.pack, st, g.leave_sms);
        default: return BRUTE_ERR_INVALID_ARG;
    }
}

}  // namespace bb

using namespace bb;

extern "C" int brute_b200_xnor_gemm(const uint64_t* A, const uint64_t* B, int32_t* C,
                                    int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                                    int impl, void* stream) {
    BB_REQUIRE(M >= 0 && N >= 0 && Kp >= 0 && K >= 0 && K <= 64 * Kp, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(K < (1ll << 30) && M < (1ll << 31) && N < (1ll << 31), BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(impl >= BRUTE_GEMM_AUTO && impl <= BRUTE_GEMM_TCGEN05_PAIR, BRUTE_ERR_INVALID_ARG);
    if (M == 0 || N == 0) return BRUTE_OK;
    BB_REQUIRE(C != nullptr && ldc >= N, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(C) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(Kp == 0 || (A != nullptr && B != nullptr), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(A) && aligned8(B), BRUTE_ERR_MISALIGNED);
    GemmArgs g{A, B, M, N, Kp, K, C, ldc, nullptr, nullptr, 0, false};
    if (Kp == 0) return run_popc(g, as_stream(stream));     // C = K (= 0) everywhere
    return dispatch(g, impl, as_stream(stream));
}

extern "C" int brute_b200_xnor_gemm_leave_sms(const uint64_t* A, const uint64_t* B, int32_t* C,
                                              int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                                              int leave_sms, void* stream) {
    BB_REQUIRE(M >= 0 && N >= 0 && Kp >= 0 && K >= 0 && K <= 64 * Kp, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(K < (1ll << 30) && M < (1ll << 31) && N < (1ll << 31), BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(leave_sms >= 0 && leave_sms <= kNumSMs - 2, BRUTE_ERR_INVALID_ARG);
    if (M == 0 || N == 0) return BRUTE_OK;
    BB_REQUIRE(C != nullptr && ldc >= N, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(C) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(Kp == 0 || (A != nullptr && B != nullptr), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(A) && aligned8(B), BRUTE_ERR_MISALIGNED);
    GemmArgs g{A, B, M, N, Kp, K, C, ldc, nullptr, nullptr, 0, false};
    g.leave_sms = leave_sms;
    if (Kp == 0) return run_popc(g, as_stream(stream));
    return dispatch(g, BRUTE_GEMM_AUTO, as_stream(stream));
}

extern "C" int brute_b200_xnor_gemm_i16(const uint64_t* A, const uint64_t* B, int16_t* C,
                                        int64_t M, int64_t N, int64_t Kp, int64_t K, int64_t ldc,
                                        int leave_sms, void* stream) {
    BB_REQUIRE(M >= 0 && N >= 0 && Kp >= 0 && K >= 0 && K <= 64 * Kp, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(K <= 32767 && Kp > 0 && M < (1ll << 31) && N < (1ll << 31), BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(leave_sms >= 0 && leave_sms <= kNumSMs - 2, BRUTE_ERR_INVALID_ARG);
    if (M == 0 || N == 0) return BRUTE_OK;
    BB_REQUIRE(C != nullptr && ldc >= N && A != nullptr && B != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE((reinterpret_cast<uintptr_t>(C) & 1u) == 0 && aligned8(A) && aligned8(B), BRUTE_ERR_MISALIGNED);
    return tc5_pair_run_i16(A, B, M, N, Kp, K, C, ldc, as_stream(stream), leave_sms);
}

extern "C" int brute_b200_xnor_gemm_scale_sign_pack(const uint64_t* A, const uint64_t* B,
                                                    const float* scale, uint64_t* out,
                                                    int64_t M, int64_t N, int64_t Kp, int64_t K,
                                                    int mode, int impl, void* stream) {
    BB_REQUIRE(M >= 0 && N >= 0 && Kp >= 0 && K >= 0 && K <= 64 * Kp, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(K < (1ll << 30) && M < (1ll << 31) && N < (1ll << 31), BRUTE_ERR_UNSUPPORTED);
    BB_REQUIRE(mode == BRUTE_SIGN_GT0 || mode == BRUTE_SIGN_GE0, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(impl >= BRUTE_GEMM_AUTO && impl <= BRUTE_GEMM_TCGEN05_PAIR, BRUTE_ERR_INVALID_ARG);
    if (M == 0 || N == 0) return BRUTE_OK;
    BB_REQUIRE(scale != nullptr && out != nullptr, BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(out) && (reinterpret_cast<uintptr_t>(scale) & 3u) == 0, BRUTE_ERR_MISALIGNED);
    BB_REQUIRE(Kp == 0 || (A != nullptr && B != nullptr), BRUTE_ERR_INVALID_ARG);
    BB_REQUIRE(aligned8(A) && aligned8(B), BRUTE_ERR_MISALIGNED);
    GemmArgs g{A, B, M, N, Kp, K, nullptr, 0, scale, out, mode, true};
    if (Kp == 0) return run_popc(g, as_stream(stream));
    return dispatch(g, impl, as_stream(stream));
}

namespace bb { int tc5_status_bridge() { return tc5_device_status(); } }

// ---------------------------------------------------------------------------
// Self-test of the bounded wait that every tcgen05 kernel of the library relies on: one CTA waits,
// with a SHORT limit, on an mbarrier that nothing will ever arrive at. The wait must give up, record
// its code in the status word and let the kernel return; nothing traps and nothing spins forever.
namespace bb {
constexpr int TC_CODE_SELFTEST = 99;
__global__ void k_selftest_bounded_wait(uint64_t limit_ns, int relaxed, int* gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init((uint32_t)__cvta_generic_to_shared(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar);
        const bool ok = relaxed ? mbar_wait_limit<true>(b, 0, &abort_flag, TC_CODE_SELFTEST, limit_ns)
                                : mbar_wait_limit<false>(b, 0, &abort_flag, TC_CODE_SELFTEST, limit_ns);
        *gave_up = ok ? 0 : 1;
    }
    __syncthreads();
    // the other threads see the abort flag, as the roles of a real kernel do
    if (threadIdx.x == 32 && abort_flag) atomicAdd(gave_up, 2);
}
}  // namespace bb

extern "C" int brute_b200_selftest_bounded_wait(int64_t limit_us, int relaxed, int* gave_up_device, void* stream) {
    BB_REQUIRE(limit_us >= 1 && limit_us <= 100000 && gave_up_device != nullptr, BRUTE_ERR_INVALID_ARG);
    k_selftest_bounded_wait<<<1, 64, 0, as_stream(stream)>>>((uint64_t)limit_us * 1000ull, relaxed, gave_up_device);
    return launch_status();
}
