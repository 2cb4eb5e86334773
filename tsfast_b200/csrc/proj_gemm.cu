// Boundary projections of the diagonal-scan layers (LRU / S5) on the 5th-generation tensor cores:
//   C[M, N] = A1[M, K1] * B1[N, K1]^T  (+ A2[M, K2] * B2[N, K2]^T),   float32 in, float32 out.
// M is the token axis (batch x time, hundreds of thousands of rows), K and N are feature widths
// (tens to hundreds), so each product is a skinny GEMM whose cost is reading A and writing C once;
// the only reason it is slow as a float32 SIMT GEMM is arithmetic.  Here the arithmetic runs as
// tcgen05.mma.kind::tf32 with float32-faithful numerics: every operand is split x = hi + lo with hi
// the value truncated to TF32 (10 mantissa bits kept) and lo = x - hi (exact in float32), and the
// product is accumulated in float32 in tensor memory as  hi*hi + hi*lo + lo*hi  (the dropped lo*lo
// term is below 2^-22 relative).
//
// One CTA (128 threads) computes one 128 x 128 tile of C:
//   * thread 0 asks the TMA unit for the next K-block (32 floats = one 128-byte swizzle row) of A and
//     of the two halves of B, which land in shared memory in the 128-byte-swizzled K-major layout the
//     tensor core reads (cp.async.bulk.tensor, completion on an mbarrier);
//   * all threads split the A block in place into hi and lo (elementwise, so the swizzle is irrelevant);
//   * thread 0 issues the 4 x 3 MMAs of the block (K = 8 per instruction) and commits them to a second
//     mbarrier; the accumulator [128 lanes x 128 columns] lives in tensor memory;
//   * after the last block each warp reads its 32 lanes with tcgen05.ld, stages them in shared memory
//     and stores whole 512-byte rows.
// Shared memory per CTA is 64 KB and the accumulator 128 of the 512 tensor-memory columns, so three
// CTAs share an SM and overlap one another's copy, split, MMA and store phases.
// The weights' halves are prepared once per call by split_weights_kernel into the caller's workspace.
// Every wait on an mbarrier is bounded; a wait that runs out records B200_ERR_TIMEOUT in the
// workspace header, and the CTA still frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace b200 {

constexpr int kBM = 128;       // rows of C per CTA (= tensor-memory lanes)
constexpr int kBN = 128;       // columns of C per CTA (= tensor-memory columns, MMA N)
constexpr int kBK = 32;        // floats per K-block: one 128-byte swizzle row
constexpr int kTileBytes = kBM * kBK * 4;  // 16 KB: one operand block
constexpr int kGemmSmem = 4 * kTileBytes + 1024;  // A(hi), A lo, B hi, B lo + alignment slack
constexpr int kWaitLimit = 200000;  // polls of an mbarrier (about 100 ns apart) before a wait gives up: tens of ms

struct ProjArgs {
    float* C;
    long long ldc;
    long long M, N;
    int kb1, kb2;  // K-blocks of the first and of the second product
    WsHeader* hdr;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false when the poll limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// Shared-memory matrix descriptor of a K-major operand block in the 128-byte-swizzled layout: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major), 16 B
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;             // descriptor version
    d |= (uint64_t)2 << 61;             // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B TF32, both K-major, M = 128, N = kBN.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// x = hi + lo with hi = x truncated to TF32 (sign, 8 exponent and 10 mantissa bits)
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
    hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    lo = x - hi;
}

// B[N, K] (row pitch ldb) -> hi[N, K], lo[N, K] dense
__global__ void split_weights_kernel(const float* __restrict__ B, long long ldb, long long N, long long K,
                                     float* __restrict__ hi, float* __restrict__ lo) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * K) return;
    const long long r = i / K, c = i - r * K;
    float h, l;
    split_tf32(B[r * ldb + c], h, l);
    hi[i] = h;
    lo[i] = l;
}

__global__ void __launch_bounds__(128, 3)
proj_gemm_kernel(const __grid_constant__ CUtensorMap mapA1, const __grid_constant__ CUtensorMap mapB1hi,
                 const __grid_constant__ CUtensorMap mapB1lo, const __grid_constant__ CUtensorMap mapA2,
                 const __grid_constant__ CUtensorMap mapB2hi, const __grid_constant__ CUtensorMap mapB2lo,
                 const ProjArgs p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_tma, bar_mma;
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
    // 1024-byte aligned operand blocks (the swizzle pattern repeats every 1024 bytes)
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* sA = reinterpret_cast<float*>(base);
    float* sAlo = reinterpret_cast<float*>(base + kTileBytes);
    float* sBhi = reinterpret_cast<float*>(base + 2 * kTileBytes);
    float* sBlo = reinterpret_cast<float*>(base + 3 * kTileBytes);

    const long long n_tiles = (p.N + kBN - 1) / kBN;
    const long long m_tile = blockIdx.x / n_tiles, n_tile = blockIdx.x - m_tile * n_tiles;
    const int row0 = (int)(m_tile * kBM), col0 = (int)(n_tile * kBN);

    if (tid == 0) {
        mbar_init(&bar_tma, 1);
        mbar_init(&bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 1) {  // one warp allocates the accumulator columns and gives up the right to allocate more
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kBN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    // `ok` is uniform over the CTA (it comes out of a barrier vote), so a wait that ran out takes every
    // thread out of the loop together and no barrier is left half-attended
    int ok = 1;
    const int nkb = p.kb1 + p.kb2;
    for (int kb = 0; kb < nkb && ok; ++kb) {
        const uint32_t parity = (uint32_t)(kb & 1);
        if (tid == 0) {
            const bool first = kb < p.kb1;
            const int kx = (first ? kb : kb - p.kb1) * kBK;
            mbar_expect_tx(&bar_tma, 3 * kTileBytes);
            tma_load_2d(sA, first ? &mapA1 : &mapA2, kx, row0, &bar_tma);
            tma_load_2d(sBhi, first ? &mapB1hi : &mapB2hi, kx, col0, &bar_tma);
            tma_load_2d(sBlo, first ? &mapB1lo : &mapB2lo, kx, col0, &bar_tma);
        }
        const int landed = mbar_wait(&bar_tma, parity) ? 1 : 0;
        // split the A block: hi in place, lo beside it (same swizzled position)
#pragma unroll
        for (int j = 0; j < kTileBytes / 16 / 128; ++j) {
            float4 x = reinterpret_cast<float4*>(sA)[j * 128 + tid];
            float4 h, l;
            split_tf32(x.x, h.x, l.x), split_tf32(x.y, h.y, l.y), split_tf32(x.z, h.z, l.z), split_tf32(x.w, h.w, l.w);
            reinterpret_cast<float4*>(sA)[j * 128 + tid] = h;
            reinterpret_cast<float4*>(sAlo)[j * 128 + tid] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        ok = __syncthreads_and(landed);
        if (ok) {
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dA = umma_desc_k_sw128(smem_u32(sA)), dAl = umma_desc_k_sw128(smem_u32(sAlo));
                const uint64_t dBh = umma_desc_k_sw128(smem_u32(sBhi)), dBl = umma_desc_k_sw128(smem_u32(sBlo));
#pragma unroll
                for (int k = 0; k < kBK / 8; ++k) {  // 8 floats = 32 bytes per MMA along K: +2 in 16-byte units
                    const uint64_t adv = (uint64_t)(2 * k);
                    umma_tf32(tmem_d, dAl + adv, dBh + adv, (kb | k) != 0);
                    umma_tf32(tmem_d, dA + adv, dBl + adv, 1u);
                    umma_tf32(tmem_d, dA + adv, dBh + adv, 1u);
                }
                umma_commit(&bar_mma);
            }
            // the MMAs have read the blocks once this completes: only then may they be overwritten
            ok = __syncthreads_and(mbar_wait(&bar_mma, parity) ? 1 : 0);
        }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (ok) {
        // epilogue: warp w owns accumulator lanes (rows) 32w .. 32w+31; 32 columns at a time go through a
        // padded shared-memory patch so that every store instruction writes whole 128-byte row pieces
        float* patch = reinterpret_cast<float*>(base) + wid * (32 * 36);
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
            float v[32];
            tmem_ld32(tmem_d + ((uint32_t)(wid * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(patch + lane * 36 + q * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            __syncwarp();
            const int cc = (lane & 7) * 4;  // 8 lanes cover one row piece of 32 columns
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                const int r = rr * 4 + (lane >> 3);
                const long long grow = (long long)row0 + wid * 32 + r;
                const long long gcol = (long long)col0 + c * 32 + cc;
                if (grow < p.M && gcol < p.N) {
                    const float4 o = *reinterpret_cast<const float4*>(patch + r * 36 + cc);
                    float* dst = p.C + grow * p.ldc + gcol;
                    if (gcol + 3 < p.N) {
                        __stcs(reinterpret_cast<float4*>(dst), o);
                    } else {
                        const float ov[4] = {o.x, o.y, o.z, o.w};
                        for (int e = 0; e < 4 && gcol + e < p.N; ++e) dst[e] = ov[e];
                    }
                }
            }
            __syncwarp();
        }
    } else if (tid == 0) {
        atomicExch(&p.hdr->error, (unsigned int)B200_ERR_TIMEOUT);
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // give copies still in flight a bounded time to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kBN) : "memory");
    }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Tensor map of a row-major float32 matrix [rows, cols] (row pitch ld floats) read in boxes of
// kBK columns x 128 rows into the 128-byte-swizzled layout; rows and columns past the end read as zero.
static bool make_map(CUtensorMap* map, const float* ptr, long long rows, long long cols, long long ld) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct ProjWs {
    size_t off_b1hi, off_b1lo, off_b2hi, off_b2lo, total;
};
static ProjWs proj_ws(long long N, long long K1, long long K2) {
    ProjWs w;
    size_t off = align_up(sizeof(WsHeader), 256);
    const size_t s1 = align_up(sizeof(float) * (size_t)(N * K1), 256), s2 = align_up(sizeof(float) * (size_t)(N * K2), 256);
    w.off_b1hi = off, off += s1;
    w.off_b1lo = off, off += s1;
    w.off_b2hi = off, off += s2;
    w.off_b2lo = off, off += s2;
    w.total = off;
    return w;
}

static bool row_ok(const void* p, long long ld) { return p != nullptr && ((uintptr_t)p & 15) == 0 && ld % 4 == 0; }

}  // namespace b200

extern "C" {

size_t b200_proj_gemm_workspace_bytes(int64_t N, int64_t K1, int64_t K2) {
    if (N <= 0 || K1 < 0 || K2 < 0) return 256;
    return b200::proj_ws(N, K1, K2).total;
}

int b200_proj_gemm(int64_t M, int64_t N, int64_t K1, const void* A1, int64_t lda1, const void* B1, int64_t ldb1,
                   int64_t K2, const void* A2, int64_t lda2, const void* B2, int64_t ldb2, void* C, int64_t ldc,
                   void* workspace, size_t workspace_bytes, void* stream) {
    using namespace b200;
    if (M < 0 || N <= 0 || K1 <= 0 || K2 < 0) return B200_ERR_ARG;
    if (M == 0) return B200_OK;
    if (K1 % kBK != 0 || K2 % kBK != 0) return B200_ERR_UNSUPPORTED;
    if (!row_ok(A1, lda1) || !B1 || !C || ldc < N || lda1 < K1 || ldb1 < K1) return B200_ERR_ARG;
    if (K2 > 0 && (!row_ok(A2, lda2) || !B2 || lda2 < K2 || ldb2 < K2)) return B200_ERR_ARG;
    if (((uintptr_t)C & 15) != 0 || ldc % 4 != 0) return B200_ERR_ARG;
    const ProjWs w = proj_ws(N, K1, K2);
    if (!workspace || ((uintptr_t)workspace % 256) != 0 || workspace_bytes < w.total) return B200_ERR_WORKSPACE;
    const long long tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    if (tiles > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* base = static_cast<char*>(workspace);
    if (cudaMemsetAsync(base, 0, sizeof(WsHeader), st) != cudaSuccess) return B200_ERR_LAUNCH;
    float* b1hi = (float*)(base + w.off_b1hi);
    float* b1lo = (float*)(base + w.off_b1lo);
    float* b2hi = (float*)(base + w.off_b2hi);
    float* b2lo = (float*)(base + w.off_b2lo);
    split_weights_kernel<<<(unsigned int)((N * K1 + 255) / 256), 256, 0, st>>>((const float*)B1, ldb1, N, K1, b1hi, b1lo);
    if (K2 > 0)
        split_weights_kernel<<<(unsigned int)((N * K2 + 255) / 256), 256, 0, st>>>((const float*)B2, ldb2, N, K2, b2hi, b2lo);
    if (cudaGetLastError() != cudaSuccess) return B200_ERR_LAUNCH;

    CUtensorMap mA1, mB1h, mB1l, mA2, mB2h, mB2l;
    bool ok = make_map(&mA1, (const float*)A1, M, K1, lda1) && make_map(&mB1h, b1hi, N, K1, K1) && make_map(&mB1l, b1lo, N, K1, K1);
    if (K2 > 0) {
        ok = ok && make_map(&mA2, (const float*)A2, M, K2, lda2) && make_map(&mB2h, b2hi, N, K2, K2) && make_map(&mB2l, b2lo, N, K2, K2);
    } else {
        mA2 = mA1, mB2h = mB1h, mB2l = mB1l;
    }
    if (!ok) return B200_ERR_LAUNCH;

    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(proj_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) != cudaSuccess)
            return B200_ERR_LAUNCH;
        configured[dev] = true;
    }
    ProjArgs a;
    a.C = (float*)C, a.ldc = ldc, a.M = M, a.N = N;
    a.kb1 = (int)(K1 / kBK), a.kb2 = (int)(K2 / kBK);
    a.hdr = reinterpret_cast<WsHeader*>(base);
    proj_gemm_kernel<<<(unsigned int)tiles, 128, kGemmSmem, st>>>(mA1, mB1h, mB1l, mA2, mB2h, mB2l, a);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // extern "C"
