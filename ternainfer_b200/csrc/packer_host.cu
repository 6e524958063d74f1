// Host-side weight packer of libternaspmm.so (B200 tile order), the unpacker,
// and the transcoder from arrays written by the reference's packer.
//
// Format (same four arrays, element types and sizes as the reference's
// convert/convert_utils.py:52-228 and kernels/TernaSpMM.cu:282-439):
//   bitmap          u64[N*K/64]   1 bit per weight, 64 u64 (= 128 u32) per 64x64 tile
//   tile_offsets    i32[tiles+1]  prefix sums of the per-tile non-zero counts, each
//                                 rounded up to a multiple of 32 ("values" = bits)
//   quarter_offsets u16[3*tiles]  non-zeros of the tile before bit 1024, 2048, 3072
//   sign_words      u32[]         sign bit (1 = -1) of every non-zero in bit order,
//                                 LSB first, each tile zero-padded to 32 bits
// Tiles are ordered row-tile major, k-tile minor.  Inside a tile, bit index
//   b = lane*128 + word*32 + nibble*4 + e,  lane = 4g+q
// addresses weight  row = 16*word + g + 8*(nibble&1),
//                   k   = 16*q + 8*(nibble>>2) + 4*((nibble>>1)&1) + e,
// so that one lane's 16 bytes decode directly into the int8 MMA A fragments
// of four 16-row groups, and one lane's four nibbles of a row are 16
// consecutive k (one 128-bit shared-memory store on the large-batch path).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

namespace {

inline void bit_to_coord(int b, int& row, int& k) {
    const int lane = b >> 7, word = (b >> 5) & 3, nib = (b >> 2) & 7, e = b & 3;
    const int g = lane >> 2, q = lane & 3;
    row = 16 * word + g + 8 * (nib & 1);
    k = 16 * q + 8 * (nib >> 2) + 4 * ((nib >> 1) & 1) + e;
}

// Position of (row, k) of a tile in the reference's order: the matrix is first
// permuted inside 16x16 blocks into mma.m16n8k16 A-fragment order, then walked
// as 16-row warp tiles > 16-wide k groups > 2x2 8x8 blocks column-major > 8x8
// row-major (convert/convert_utils.py:8-49, :96-136).
inline int ref_bit_of(int row, int k) {
    const int i = row & 15, kk = k & 15;
    int ri = i, rk = (kk + 1) / 2;
    if (i < 8) {
        if (kk & 2) { ri += 8; rk -= 1; }
    } else {
        rk += 8;
        if ((kk & 2) == 0) ri -= 8; else rk -= 1;
    }
    const int med = row >> 4, lkg = k >> 4;
    const int bi = ri >> 3, r = ri & 7, bj = rk >> 3, c = rk & 7;
    return (((med * 4 + lkg) * 2 + bj) * 2 + bi) * 64 + r * 8 + c;
}

struct TileTables {
    int row[4096], k[4096], ref_bit[4096];
    TileTables() {
        for (int b = 0; b < 4096; ++b) {
            bit_to_coord(b, row[b], k[b]);
            ref_bit[b] = ref_bit_of(row[b], k[b]);
        }
    }
};
const TileTables& tables() {
    static TileTables t;
    return t;
}

// Pack one tile given its 4096 values in B200 bit order (value != 0 -> bit set,
// value < 0 -> sign bit 1).  Appends to the sign stream at bit position `pos`
// (a multiple of 32) and returns the new position.
long long pack_tile(const int8_t* v, uint32_t* bm128, uint16_t* q3, uint32_t* signs, long long pos) {
    int cnt = 0;
    for (int wd = 0; wd < 128; ++wd) {
        uint32_t m = 0;
        for (int j = 0; j < 32; ++j) {
            const int8_t x = v[wd * 32 + j];
            if (x) {
                m |= 1u << j;
                if (x < 0) signs[(pos + cnt) >> 5] |= 1u << ((pos + cnt) & 31);
                ++cnt;
            }
        }
        bm128[wd] = m;
        if (wd == 31) q3[0] = (uint16_t)cnt;
        if (wd == 63) q3[1] = (uint16_t)cnt;
        if (wd == 95) q3[2] = (uint16_t)cnt;
    }
    return pos + ((cnt + 31) / 32) * 32;
}

template <typename Getter>
long long pack_matrix(Getter get, int N, int K, uint64_t* bitmap, int* tile_off, uint16_t* q_off, uint32_t* signs) {
    if (N <= 0 || K <= 0 || (N % 64) || (K % 64)) return -1;
    const TileTables& T = tables();
    const int RT = N / 64, KT = K / 64;
    memset(signs, 0, ((size_t)N * K / 32 + 4) * sizeof(uint32_t));
    long long pos = 0;
    tile_off[0] = 0;
    int8_t v[4096];
    for (int rt = 0; rt < RT; ++rt)
        for (int kt = 0; kt < KT; ++kt) {
            const size_t t = (size_t)rt * KT + kt;
            for (int b = 0; b < 4096; ++b) v[b] = get((size_t)(rt * 64 + T.row[b]) * K + kt * 64 + T.k[b]);
            pos = pack_tile(v, reinterpret_cast<uint32_t*>(bitmap) + t * 128, q_off + 3 * t, signs, pos);
            tile_off[t + 1] = (int)pos;
        }
    return pos / 32;
}

}  // namespace

extern "C" long long ternaspmm_pack_i8(const int8_t* W, int N, int K, uint64_t* bitmap, int* tile_offsets,
                                       uint16_t* quarter_offsets, uint32_t* sign_words) {
    if (!W || !bitmap || !tile_offsets || !quarter_offsets || !sign_words) return -1;
    return pack_matrix([W](size_t i) { return W[i]; }, N, K, bitmap, tile_offsets, quarter_offsets, sign_words);
}

extern "C" int ternaspmm_unpack_i8(const uint64_t* bitmap, const int* tile_offsets, const uint32_t* sign_words, int N,
                                   int K, int8_t* W) {
    if (!W || !bitmap || !tile_offsets || !sign_words || N <= 0 || K <= 0 || (N % 64) || (K % 64)) return -1;
    const TileTables& T = tables();
    const int RT = N / 64, KT = K / 64;
    const uint32_t* bm = reinterpret_cast<const uint32_t*>(bitmap);
    for (int rt = 0; rt < RT; ++rt)
        for (int kt = 0; kt < KT; ++kt) {
            const size_t t = (size_t)rt * KT + kt;
            long long pos = tile_offsets[t];
            for (int b = 0; b < 4096; ++b) {
                int8_t x = 0;
                if ((bm[t * 128 + (b >> 5)] >> (b & 31)) & 1u) {
                    x = ((sign_words[pos >> 5] >> (pos & 31)) & 1u) ? -1 : 1;
                    ++pos;
                }
                W[(size_t)(rt * 64 + T.row[b]) * K + kt * 64 + T.k[b]] = x;
            }
        }
    return 0;
}

extern "C" int ternaspmm_transcode_reference_layout(const uint64_t* ref_bitmap, const int* tile_offsets,
                                                    const uint32_t* ref_sign_words, int N, int K,
                                                    uint64_t* out_bitmap, uint16_t* out_quarter_offsets,
                                                    uint32_t* out_sign_words) {
    if (!ref_bitmap || !tile_offsets || !ref_sign_words || !out_bitmap || !out_quarter_offsets || !out_sign_words ||
        N <= 0 || K <= 0 || (N % 64) || (K % 64))
        return -1;
    const TileTables& T = tables();
    const size_t tiles = (size_t)(N / 64) * (K / 64);
    const uint32_t* rbm = reinterpret_cast<const uint32_t*>(ref_bitmap);
    int8_t ref_v[4096], v[4096];
    memset(out_sign_words, 0, (size_t)tile_offsets[tiles] / 8);
    for (size_t t = 0; t < tiles; ++t) {
        long long pos = tile_offsets[t];
        for (int b = 0; b < 4096; ++b) {
            int8_t x = 0;
            if ((rbm[t * 128 + (b >> 5)] >> (b & 31)) & 1u) {
                x = ((ref_sign_words[pos >> 5] >> (pos & 31)) & 1u) ? -1 : 1;
                ++pos;
            }
            ref_v[b] = x;
        }
        for (int b = 0; b < 4096; ++b) v[b] = ref_v[T.ref_bit[b]];
        const long long end = pack_tile(v, reinterpret_cast<uint32_t*>(out_bitmap) + t * 128,
                                        out_quarter_offsets + 3 * t, out_sign_words, tile_offsets[t]);
        if (end != tile_offsets[t + 1]) return -1;
    }
    return 0;
}

extern "C" void reorder_WT_h(__nv_bfloat16* W, __nv_bfloat16* W_reordered, int N, int K) {
    if (W && W_reordered && W != W_reordered) memcpy(W_reordered, W, (size_t)N * K * sizeof(__nv_bfloat16));
}

extern "C" int convert_reorderd(__nv_bfloat16* W, int N, int K, int tile_N, int warp_subtile_N, int subtile_N,
                                int tile_K, int warp_subtile_K, int subtile_K, uint64_t** bitmap, int** tile_offsets,
                                uint16_t** quarter_offsets, uint32_t** sign_words, int* max_nnz) {
    if (!W || !bitmap || !tile_offsets || !quarter_offsets || !sign_words || !max_nnz) return -1;
    if (tile_N != 64 || warp_subtile_N != 16 || subtile_N != 8 || tile_K != 64 || warp_subtile_K != 64 ||
        subtile_K != 8 || N <= 0 || K <= 0 || (N % 64) || (K % 64))
        return -1;
    const size_t tiles = (size_t)(N / 64) * (K / 64);
    *sign_words = (uint32_t*)malloc(((size_t)N * K / 32 + 4) * sizeof(uint32_t));
    *tile_offsets = (int*)malloc((tiles + 1) * sizeof(int));
    *quarter_offsets = (uint16_t*)calloc(3 * tiles + 8, sizeof(uint16_t));
    *bitmap = nullptr;
    if (cudaMallocHost((void**)bitmap, (size_t)N * K / 8) != cudaSuccess) *bitmap = nullptr;
    if (!*sign_words || !*tile_offsets || !*quarter_offsets || !*bitmap) return -1;
    const unsigned short* raw = reinterpret_cast<const unsigned short*>(W);
    auto get = [raw](size_t i) -> int8_t {
        const unsigned short h = raw[i];
        if ((h & 0x7FFF) == 0) return 0;
        return (h & 0x8000) ? -1 : 1;
    };
    const long long words = pack_matrix(get, N, K, *bitmap, *tile_offsets, *quarter_offsets, *sign_words);
    if (words < 0) return -1;
    int mx = 0;
    for (size_t t = 0; t < tiles; ++t) {
        const int c = (*tile_offsets)[t + 1] - (*tile_offsets)[t];
        if (c > mx) mx = c;
    }
    *max_nnz = mx;
    return (int)tiles;
}
