// Layout-agnostic kernels: bit-exact dequant, the any-shape GEMV, and the repack.
//
// These accept every supported format in either device layout and make no
// alignment assumption (byte loads only).  They are the correctness floor:
// cuda_gemv uses them for shapes the streaming kernels in gemv_stream.cuh do not
// take (in_dim not a multiple of 64, unaligned base pointers, formats without a
// streaming kernel yet).
#pragma once

#include "formats.cuh"

namespace qz {

// ---- dequant to f32 (bit-exact against src/dequant.rs dequant()) ------------
template <uint32_t T, bool PLANES>
__global__ void dequant_kernel(const uint8_t *__restrict__ data, float *__restrict__ out, int K, long long n_sub,
                               const int *__restrict__ row_sel)
{
    const FormatInfo fi = format_info(T);
    pdl_wait();
    pdl_trigger();
    long long gs = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gs >= n_sub) return;
    const int subs_per_row = K / 32;
    const int subs_per_blk = fi.block_elems / 32;
    long long row = gs / subs_per_row;
    int s = (int)(gs % subs_per_row);
    int nb = K / fi.block_elems;
    // row_sel: output row r decodes source row row_sel[r], read from device memory (token ids of a recorded
    // decode step or of a prompt)
    const long long src_row = row_sel ? (long long)row_sel[row] : row;
    const uint8_t *rowp = data + (size_t)src_row * nb * fi.block_bytes;
    Fields F = block_fields<PLANES>(fi, rowp, nb, s / subs_per_blk);
    float w[32];
    decode32<T>(F, s % subs_per_blk, w);
    float *o = out + gs * 32;
#pragma unroll
    for (int i = 0; i < 32; i++) o[i] = w[i];
}

// src/dequant.rs:1321-1371 (F32 copy, F16 widen, BF16 shift)
__global__ void dequant_plain_kernel(const uint8_t *__restrict__ data, float *__restrict__ out, uint32_t type,
                                     long long n, const int *__restrict__ row_sel, int K)
{
    pdl_wait();
    pdl_trigger();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    long long j = i;   // source element
    if (row_sel) j = (long long)row_sel[i / K] * K + i % K;
    if (type == T_F32) {
        out[i] = __uint_as_float(ld_u32_bytes(data + 4 * j));
    } else if (type == T_F16) {
        out[i] = h2f(ld_u16(data + 2 * j));
    } else {
        out[i] = __uint_as_float((uint32_t)ld_u16(data + 2 * j) << 16);
    }
}

// ---- any-shape GEMV: one warp per output row --------------------------------
// Lanes stride over 32-weight groups, so all 32 lanes work whatever K is.
template <uint32_t T, bool PLANES>
__global__ void __launch_bounds__(128) gemv_generic_kernel(const uint8_t *__restrict__ W, const float *__restrict__ x,
                                                           float *__restrict__ y, int K, int N)
{
    const FormatInfo fi = format_info(T);
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= N) return;
    const int nb = K / fi.block_elems;
    const int subs_per_blk = fi.block_elems / 32;
    const uint8_t *rowp = W + (size_t)row * nb * fi.block_bytes;
    float acc = 0.f;
    for (int s = lane; s < K / 32; s += 32) {
        Fields F = block_fields<PLANES>(fi, rowp, nb, s / subs_per_blk);
        float w[32];
        decode32<T>(F, s % subs_per_blk, w);
        const float *xs = x + 32 * s;
#pragma unroll
        for (int i = 0; i < 32; i++) acc = fmaf(__ldg(xs + i), w[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = acc;
}

// F32 / F16 / BF16 rows (router weights, unquantized heads): one warp per row.
template <uint32_t T>
__global__ void __launch_bounds__(128) gemv_plain_kernel(const uint8_t *__restrict__ W, const float *__restrict__ x,
                                                         float *__restrict__ y, int K, int N)
{
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= N) return;
    constexpr int ES = (T == T_F32) ? 4 : 2;
    const uint8_t *rowp = W + (size_t)row * K * ES;
    float acc = 0.f;
    const bool vec = (K % 8 == 0) && (((uintptr_t)rowp & 15) == 0) && (((uintptr_t)x & 15) == 0);
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            float4 xa = __ldg((const float4 *)(x + k)), xb = __ldg((const float4 *)(x + k + 4));
            float wv[8];
            if (T == T_F32) {
                uint4 a = ld_stream(rowp + 4 * k), b = ld_stream(rowp + 4 * k + 16);
                wv[0] = __uint_as_float(a.x); wv[1] = __uint_as_float(a.y);
                wv[2] = __uint_as_float(a.z); wv[3] = __uint_as_float(a.w);
                wv[4] = __uint_as_float(b.x); wv[5] = __uint_as_float(b.y);
                wv[6] = __uint_as_float(b.z); wv[7] = __uint_as_float(b.w);
            } else {
                uint4 a = ld_stream(rowp + 2 * k);
                uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (T == T_F16) {
                        wv[2 * i] = h2f((uint16_t)(u[i] & 0xFFFF));
                        wv[2 * i + 1] = h2f((uint16_t)(u[i] >> 16));
                    } else {
                        wv[2 * i] = __uint_as_float(u[i] << 16);
                        wv[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
                    }
                }
            }
            acc = fmaf(xa.x, wv[0], acc); acc = fmaf(xa.y, wv[1], acc);
            acc = fmaf(xa.z, wv[2], acc); acc = fmaf(xa.w, wv[3], acc);
            acc = fmaf(xb.x, wv[4], acc); acc = fmaf(xb.y, wv[5], acc);
            acc = fmaf(xb.z, wv[6], acc); acc = fmaf(xb.w, wv[7], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            float wv;
            if (T == T_F32) wv = __uint_as_float(ld_u32_bytes(rowp + 4 * k));
            else if (T == T_F16) wv = h2f(ld_u16(rowp + 2 * k));
            else wv = __uint_as_float((uint32_t)ld_u16(rowp + 2 * k) << 16);
            acc = fmaf(__ldg(x + k), wv, acc);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = acc;
}

// ---- repack: raw blocks <-> field planes, in place, one CTA per row ----------
// The whole row is staged in shared memory, so every row is rewritten
// independently and the matrix keeps its size and row starts.
template <bool TO_PLANES>
__global__ void repack_rows_kernel(uint8_t *__restrict__ data, FormatInfo fi, int nb, long long n_rows)
{
    extern __shared__ uint8_t stage[];
    const int row_bytes = nb * fi.block_bytes;
    for (long long row = blockIdx.x; row < n_rows; row += gridDim.x) {
        uint8_t *rowp = data + (size_t)row * row_bytes;
        for (int i = threadIdx.x; i < row_bytes; i += blockDim.x) stage[i] = rowp[i];
        __syncthreads();
        // destination byte i of the new layout takes source byte src(i) of the old one
        for (int i = threadIdx.x; i < row_bytes; i += blockDim.x) {
            int raw_idx, plane_idx;
            if (TO_PLANES) {
                // i indexes the plane layout: find the field, block and byte
                plane_idx = i;
                int f = 0;
#pragma unroll
                for (int j = 1; j < 5; j++)
                    if (j < fi.nfields && i >= nb * fi.off[j]) f = j;
                int r = i - nb * fi.off[f];
                int b = r / fi.size[f], o = r % fi.size[f];
                raw_idx = b * fi.block_bytes + fi.off[f] + o;
                rowp[plane_idx] = stage[raw_idx];
            } else {
                raw_idx = i;
                int b = i / fi.block_bytes, o = i % fi.block_bytes;
                int f = 0;
#pragma unroll
                for (int j = 1; j < 5; j++)
                    if (j < fi.nfields && o >= fi.off[j]) f = j;
                plane_idx = nb * fi.off[f] + b * fi.size[f] + (o - fi.off[f]);
                rowp[raw_idx] = stage[plane_idx];
            }
        }
        __syncthreads();
    }
}

}  // namespace qz
