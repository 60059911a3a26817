// K1: qf.unpack as a stand-alone kernel, and the materialising qf.dequant(qf.unpack(w)).
//
// Both are streaming kernels bound by HBM: unpack reads 1 byte and writes 2 per input byte;
// dequant reads 0.5 byte and writes 2 per weight.  Each thread moves 16 input bytes with one
// 128-bit load and writes them back with 128-bit stores.
#include "qf_common.cuh"

namespace qf {

// 4 packed bytes -> 8 output bytes.  lo = low nibbles, hi = high nibbles (one per byte lane);
// prmt interleaves them: (lo.b0, hi.b0, lo.b1, hi.b1) and (lo.b2, hi.b2, lo.b3, hi.b3).
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t &o0, uint32_t &o1) {
    const uint32_t lo = w & 0x0f0f0f0fu;
    const uint32_t hi = (w >> 4) & 0x0f0f0f0fu;
    o0 = prmt(lo, hi, 0x5140u);
    o1 = prmt(lo, hi, 0x7362u);
}

__global__ void __launch_bounds__(256) unpack_vec_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out,
                                                         int64_t n_vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        uint4 v;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(in + i));
        uint4 a, b;
        unpack_word(v.x, a.x, a.y);
        unpack_word(v.y, a.z, a.w);
        unpack_word(v.z, b.x, b.y);
        unpack_word(v.w, b.z, b.w);
        out[2 * i] = a;
        out[2 * i + 1] = b;
    }
}

// Any byte count / alignment: one byte per thread.
__global__ void __launch_bounds__(256) unpack_byte_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out,
                                                          int64_t n_bytes) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += stride) {
        const uint8_t b = in[i];
        uchar2 o;
        o.x = b & 0x0f;
        o.y = (b >> 4) & 0x0f;
        reinterpret_cast<uchar2 *>(out)[i] = o;
    }
}

int launch_unpack(qf_ctx *ctx, const void *packed, void *out, int64_t rows, int64_t packed_cols, cudaStream_t s) {
    const int64_t n_bytes = rows * packed_cols;
    if (n_bytes == 0) return QF_OK;
    const bool vec_ok = (n_bytes % 16 == 0) && ((uintptr_t)packed % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const int sms = ctx->sm_count;
    if (vec_ok) {
        const int64_t n_vec = n_bytes / 16;
        int64_t blocks = (n_vec + 255) / 256;
        if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
        unpack_vec_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const uint4 *>(packed),
                                                          reinterpret_cast<uint4 *>(out), n_vec);
    } else {
        int64_t blocks = (n_bytes + 255) / 256;
        if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
        unpack_byte_kernel<<<(unsigned)blocks, 256, 0, s>>>(reinterpret_cast<const uint8_t *>(packed),
                                                           reinterpret_cast<uint8_t *>(out), n_bytes);
    }
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

// Nibble permutation inside each word. canonical nibbles c0..c7 -> interleaved c0 c2 c4 c6 c1 c3 c5 c7.
__device__ __forceinline__ uint32_t interleave_word(uint32_t w) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r |= ((w >> (8 * i)) & 0xFu) << (4 * i);            // even codes -> nibbles 0..3
        r |= ((w >> (8 * i + 4)) & 0xFu) << (4 * (i + 4));  // odd codes  -> nibbles 4..7
    }
    return r;
}
__device__ __forceinline__ uint32_t deinterleave_word(uint32_t w) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r |= ((w >> (4 * i)) & 0xFu) << (8 * i);
        r |= ((w >> (4 * (i + 4))) & 0xFu) << (8 * i + 4);
    }
    return r;
}

__global__ void __launch_bounds__(256) prepack_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out,
                                                      int64_t n_words, int to_canonical) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
        const uint32_t w = in[i];
        out[i] = to_canonical ? deinterleave_word(w) : interleave_word(w);
    }
}

int launch_prepack(qf_ctx *ctx, const void *in, void *out, int64_t n_words, int to_canonical, cudaStream_t s) {
    int64_t blocks = (n_words + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    prepack_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint32_t *)in, (uint32_t *)out, n_words, to_canonical);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

// canonical word (n, j) <-> tiled word ((nt * KB + kb) * 128 + r) * 16 + w, n = nt*128 + r, j = kb*16 + w.
__global__ void __launch_bounds__(256) prepack_tiled_kernel(const uint32_t *__restrict__ in,
                                                            uint32_t *__restrict__ out, int64_t N, int64_t K,
                                                            int to_canonical) {
    const int64_t words_per_row = K >> 3;
    const int64_t KB = K >> 7;
    const int64_t total = N * words_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        // i enumerates the TILED order so that the side written (or read) in bulk is contiguous
        const int64_t w = i & 15;
        const int64_t r = (i >> 4) & 127;
        const int64_t blk = i >> 11;
        const int64_t kb = blk % KB;
        const int64_t nt = blk / KB;
        const int64_t canon = (nt * 128 + r) * words_per_row + kb * 16 + w;
        if (to_canonical)
            out[canon] = deinterleave_word(in[i]);
        else
            out[i] = interleave_word(in[canon]);
    }
}

int launch_prepack_tiled(qf_ctx *ctx, const void *in, void *out, int64_t N, int64_t K, int to_canonical,
                         cudaStream_t s) {
    const int64_t total = N * (K / 8);
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    prepack_tiled_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint32_t *)in, (uint32_t *)out, N, K, to_canonical);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

// W[K, N] (one code per byte, or two per byte along N) -> canonical qweight [N, K/8] words. One thread per output
// word; consecutive threads take consecutive n, so the reads are coalesced (the 4-byte writes are not: one-time op).
__global__ void __launch_bounds__(256) repack_kn_kernel(const uint8_t *__restrict__ w_kn, int packed_along_n,
                                                        int64_t K, int64_t N, uint32_t *__restrict__ out) {
    const int64_t words_per_row = K >> 3;
    const int64_t total = N * words_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t n = i % N;
        const int64_t j = i / N;
        uint32_t word = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int64_t k = 8 * j + c;
            uint32_t code;
            if (packed_along_n) {
                const uint32_t b = w_kn[k * (N >> 1) + (n >> 1)];
                code = (n & 1) ? (b >> 4) & 0xFu : b & 0xFu;
            } else {
                code = w_kn[k * N + n] & 0xFu;
            }
            word |= code << (4 * c);
        }
        out[n * words_per_row + j] = word;
    }
}

int launch_repack_kn(qf_ctx *ctx, const void *w_kn, int packed_along_n, int64_t K, int64_t N, void *out,
                     cudaStream_t s) {
    const int64_t total = N * (K / 8);
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    repack_kn_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint8_t *)w_kn, packed_along_n, K, N, (uint32_t *)out);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

// One thread per packed word (8 codes along K of one row).
template <bool BF16, int ZMODE>
__global__ void __launch_bounds__(256) dequant_kernel(const uint32_t *__restrict__ qw,
                                                      const uint16_t *__restrict__ scales,
                                                      const void *__restrict__ zeros, int zero_const,
                                                      uint4 *__restrict__ w_out, int64_t N, int64_t K, int group) {
    const int64_t words_per_row = K >> 3;
    const int64_t total = N * words_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t n = i / words_per_row;
        const int64_t j = i - n * words_per_row;
        const int64_t gi = (j * 8) / group;
        ZeroScale<BF16> zs;
        zs.set(load_zero<ZMODE>(zeros, zero_const, gi, n, N), __ldg(scales + gi * N + n));
        uint32_t p[4];
        dequant8<BF16>(__ldg(qw + i), zs, p);
        // p[i] = (c_i, c_{i+4}) -> memory order (c0,c1)(c2,c3)(c4,c5)(c6,c7)
        uint4 o;
        o.x = prmt(p[0], p[1], 0x5410u);
        o.y = prmt(p[2], p[3], 0x5410u);
        o.z = prmt(p[0], p[1], 0x7632u);
        o.w = prmt(p[2], p[3], 0x7632u);
        w_out[i] = o;
    }
}

template <bool BF16>
static void dequant_dispatch(int zmode, unsigned blocks, cudaStream_t s, const uint32_t *qw, const uint16_t *sc,
                             const void *z, int zc, uint4 *out, int64_t N, int64_t K, int group) {
    if (zmode == QF_ZERO_CONST)
        dequant_kernel<BF16, QF_ZERO_CONST><<<blocks, 256, 0, s>>>(qw, sc, z, zc, out, N, K, group);
    else if (zmode == QF_ZERO_U4)
        dequant_kernel<BF16, QF_ZERO_U4><<<blocks, 256, 0, s>>>(qw, sc, z, zc, out, N, K, group);
    else
        dequant_kernel<BF16, QF_ZERO_I8><<<blocks, 256, 0, s>>>(qw, sc, z, zc, out, N, K, group);
}

int launch_dequant(qf_ctx *ctx, const qf_linear_desc *d, const void *qw, const void *scales, const void *zeros,
                   void *w_out, cudaStream_t s) {
    const int64_t total = d->N * (d->K / 8);
    if (total == 0) return QF_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
    if (d->act_dtype == QF_BF16)
        dequant_dispatch<true>(d->zero_mode, (unsigned)blocks, s, (const uint32_t *)qw, (const uint16_t *)scales,
                               zeros, d->zero_const, (uint4 *)w_out, d->N, d->K, d->group_size);
    else
        dequant_dispatch<false>(d->zero_mode, (unsigned)blocks, s, (const uint32_t *)qw, (const uint16_t *)scales,
                                zeros, d->zero_const, (uint4 *)w_out, d->N, d->K, d->group_size);
    g_launch_count.fetch_add(1);
    QF_CUDA_TRY(ctx, cudaGetLastError());
    return QF_OK;
}

}  // namespace qf
