// Block-scaled (MX) quant matmul on tcgen05: e8m0 scale per 32 k on both operands, applied by the tensor core.
// Included by qmm_umma.cu (same translation unit: shares the tensor-map helpers, the status word and the row store).
//
// Replaces the reference's MX kernel (matmul/common/cmct/kernel/kernel_qbmm_mx.h:137-361, block/block_mmad_mx.h:396-881;
// golden quant_batch_matmul_v3/tests/assets/qbmmv3_kernel_golden.py:153-234): out = (x1 * 2^e1) @ (x2 * 2^e2) + bias, fp32
// accumulate. MXFP8 uses kind::mxf8f6f4 (k = 32 per MMA, one scale byte per row per MMA), MXFP4 uses kind::mxf4 with
// scale_vec::2X (k = 64 per MMA, two scale bytes per row per MMA); fp4 operands must be k-contiguous (the instruction has
// no MN-major form for 4-bit data).
//
// Scale factors. The tensor core wants them in TMEM, 128 rows x 4 k-blocks as "32 lanes x 16 bytes": byte
// (row % 32) * 16 + (row / 32) * 4 + kblock. The reference keeps them as (rows, ceil(k/64), 2) or (ceil(k/64), rows, 2)
// e8m0 matrices, so a small pre-pass kernel rewrites both operands' scales into that 512-byte atom order in workspace,
// [batch][row tile][k stage][atom]; the producer then fetches a stage's atoms with one untiled bulk copy per operand next to
// the two TMA loads, and the MMA warp moves them shared -> TMEM with tcgen05.cp right before the stage's MMAs (tcgen05
// operations of one thread execute in issue order, so one TMEM slot per operand is enough).
namespace {

// Tile widths: 224 columns is the widest whose two accumulators (at TMEM columns 0 and 256) leave room for the scale
// slots (columns 224..247) in the 512 columns an SM has; 128 for narrow problems.
template <int BN>
struct MxTile {
    static constexpr int kRowAtoms = BN > 128 ? 2 : 1;            // 128-row scale atoms covering the B tile's rows
    static constexpr uint32_t kBSmem = BN > 128 ? 32768u : 16384u;  // bytes reserved for B per stage (two 128-column boxes when n-major)
    static constexpr uint32_t kAcc1Col = BN > 128 ? 256u : 128u;    // second accumulator
    static constexpr uint32_t kSfaCol = BN > 128 ? 224u : 256u;     // scale slots: A first, then B
};

// One thread per 32-bit word of the atoms: rows (tile*128 + word%4... see index math), four consecutive k-blocks.
__global__ void mx_sf_relayout_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int64_t kblocks,
                                      int64_t kq, int transposed_layout, int64_t tiles, int64_t stages, int atoms, int64_t batch,
                                      int64_t src_bs, int tile_rows, int row_atoms)
{
    // atom order in workspace: [batch][tile][stage][k atom][row atom]; a row atom is 128 consecutive rows of the tile
    const int64_t words = batch * tiles * stages * atoms * row_atoms * 128;
    for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
        const int l = (int)(w & 31), m1 = (int)((w >> 5) & 3);
        int64_t r = w >> 7;
        const int ra = (int)(r % row_atoms); r /= row_atoms;
        const int at = (int)(r % atoms); r /= atoms;
        const int64_t st = r % stages; r /= stages;
        const int64_t tile = r % tiles;
        const int64_t b = r / tiles;
        const int in_tile = ra * 128 + m1 * 32 + l;
        const int64_t row = in_tile < tile_rows ? tile * tile_rows + in_tile : rows;  // past the tile: no such row
        const int64_t kb0 = (st * atoms + at) * 4;
        const uint8_t* s = src + b * src_bs;
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t kb = kb0 + j;
            uint32_t v = 127u;  // 2^0 for rows / k-blocks that do not exist (their data is zero-filled)
            if (row < rows && kb < kblocks)
                v = transposed_layout ? s[((kb >> 1) * rows + row) * 2 + (kb & 1)] : s[row * (2 * kq) + kb];
            word |= v << (8 * j);
        }
        // destination: atom base + (row % 32) * 16 + (row / 32 % 4) * 4
        const int64_t atom_idx = (((b * tiles + tile) * stages + st) * atoms + at) * row_atoms + ra;
        *reinterpret_cast<uint32_t*>(dst + atom_idx * 512 + l * 16 + m1 * 4) = word;
    }
}

// The same relayout staged through shared memory: one CTA per (batch, tile, row atom) = 128 rows, k-blocks in chunks of 256.
// Reads follow the source's contiguous axis (row-major scales: 32-bit words along k; scales stored (k/64, rows, 2): 16-bit
// pairs along the rows), writes are whole 512-byte atoms. The per-word kernel above reads or writes 4 bytes per 32-byte
// sector; this one moves whole sectors both ways. Needs an even k/64 count for the word loads, else falls back to bytes.
constexpr int kSfChunk = 256;
__global__ void __launch_bounds__(256) mx_sf_relayout_tiled_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows,
                                                                   int64_t kblocks, int64_t kq, int transposed_layout, int64_t tiles,
                                                                   int64_t stages, int atoms, int64_t src_bs, int tile_rows, int row_atoms)
{
    __shared__ __align__(16) uint8_t sm[128][kSfChunk + 4];
    int64_t r = blockIdx.x;
    const int ra = (int)(r % row_atoms); r /= row_atoms;
    const int64_t tile = r % tiles;
    const int64_t b = r / tiles;
    const uint8_t* s = src + b * src_bs;
    const int64_t row0 = tile * tile_rows + ra * 128;                       // first row of this atom column
    const int live = (int)max((int64_t)0, min((int64_t)128, min((int64_t)tile_rows - ra * 128, rows - row0)));  // rows that exist
    const int64_t kb_total = stages * atoms * 4;                            // k-blocks the atoms cover (>= kblocks)
    const int tid = threadIdx.x;
    for (int64_t kc0 = 0; kc0 < kb_total; kc0 += kSfChunk) {
        const int kc = (int)min((int64_t)kSfChunk, kb_total - kc0);         // multiple of 4
        __syncthreads();
        const bool vec16 = !transposed_layout && ((2 * kq) & 15) == 0 && (reinterpret_cast<uintptr_t>(s) & 15) == 0 && (kc & 15) == 0 &&
                           kc0 + kc <= kblocks;
        if (vec16) {
            // whole chunk present and 16-byte aligned rows: 16 k-blocks per load, four independent loads in flight per thread
            const int vecs = kc / 16;
            for (int e0 = tid; e0 < 128 * vecs; e0 += 4 * 256) {
                uint4 v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int e = e0 + j * 256;
                    v[j] = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
                    if (e < 128 * vecs) {
                        const int rr = e / vecs, c = e - rr * vecs;
                        if (rr < live) v[j] = __ldg(reinterpret_cast<const uint4*>(s + (row0 + rr) * (2 * kq) + kc0 + 16 * c));
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int e = e0 + j * 256;
                    if (e < 128 * vecs) {
                        const int rr = e / vecs, c = e - rr * vecs;
                        uint32_t* d32 = reinterpret_cast<uint32_t*>(&sm[rr][16 * c]);
                        d32[0] = v[j].x; d32[1] = v[j].y; d32[2] = v[j].z; d32[3] = v[j].w;
                    }
                }
            }
        } else if (!transposed_layout) {
            const bool words = ((2 * kq) & 3) == 0 && (reinterpret_cast<uintptr_t>(s) & 3) == 0;
            for (int e = tid; e < 128 * (kc / 4); e += 256) {
                const int rr = e / (kc / 4), c4 = e % (kc / 4);
                const int64_t kb = kc0 + 4 * c4;
                uint32_t w = 0x7F7F7F7Fu;  // 2^0 where no row / k-block exists (the data there is zero-filled)
                if (rr < live) {
                    const uint8_t* q = s + (row0 + rr) * (2 * kq) + kb;
                    if (words && kb + 3 < kblocks) {
                        w = __ldg(reinterpret_cast<const uint32_t*>(q));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (kb + j < kblocks) w = (w & ~(0xFFu << (8 * j))) | ((uint32_t)q[j] << (8 * j));
                    }
                }
                *reinterpret_cast<uint32_t*>(&sm[rr][4 * c4]) = w;
            }
        } else {
            for (int e = tid; e < 128 * (kc / 2); e += 256) {
                const int kbp = e >> 7, rr = e & 127;   // pair of k-blocks, row: consecutive threads read consecutive rows
                const int64_t kb = kc0 + 2 * kbp;
                uint32_t w = 0x7F7Fu;
                if (rr < live && kb < kblocks) {
                    const uint8_t* q = s + ((kb >> 1) * rows + row0 + rr) * 2;
                    w = (reinterpret_cast<uintptr_t>(q) & 1) ? ((uint32_t)q[0] | ((uint32_t)q[1] << 8)) : (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(q));
                    if (kb + 1 >= kblocks) w = (w & 0xFFu) | 0x7F00u;
                }
                *reinterpret_cast<uint16_t*>(&sm[rr][2 * kbp]) = (uint16_t)w;
            }
        }
        __syncthreads();
        // atoms of this chunk: atom (st, at) holds k-blocks 4 * (st * atoms + at) .. + 3; 128 words of 4 bytes each
        const int natoms = kc / 4;
        for (int e = tid; e < natoms * 128; e += 256) {
            const int ai = e >> 7, wi = e & 127;
            const int l = wi >> 2, m1 = wi & 3, rr = m1 * 32 + l;
            const int64_t ka = kc0 / 4 + ai;              // = st * atoms + at
            const int64_t st = ka / atoms;
            const int at = (int)(ka % atoms);
            const int64_t atom_idx = (((b * tiles + tile) * stages + st) * atoms + at) * row_atoms + ra;
            *reinterpret_cast<uint32_t*>(dst + atom_idx * 512 + wi * 4) = *reinterpret_cast<const uint32_t*>(&sm[rr][4 * ai]);
        }
    }
}

// fp4 operands stored along m / n (x1 given as (k,m), x2 as (k,n)) cannot be fed to the tensor core (kind::mxf4 has no MN-major
// form); a pre-pass rewrites them k-contiguous into workspace: (R, C) packed along C -> (C, R) packed along R, two e2m1 per
// byte, low nibble first. 64 x 64 element tiles through shared memory; ~1.5 % of the matmul's time at the benchmark shape.
__global__ void __launch_bounds__(256) fp4_transpose_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t R, int64_t C,
                                                            int64_t src_pitch, int64_t dst_pitch, int64_t src_bs, int64_t dst_bs)
{
    __shared__ __align__(16) uint8_t tile[64][68];  // one element per byte
    const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
    const uint8_t* s = src + (int64_t)blockIdx.z * src_bs;
    uint8_t* d = dst + (int64_t)blockIdx.z * dst_bs;
    const int t = threadIdx.x;
    const bool whole = r0 + 64 <= R && c0 + 64 <= C && (src_pitch & 7) == 0 && (dst_pitch & 7) == 0 &&
                       ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 7) == 0;
    {
        const int row = t >> 2, seg = t & 3;  // 8 source bytes = 16 elements of one row
        const int64_t r = r0 + row;
        if (whole) {
            const uint2 v = *reinterpret_cast<const uint2*>(s + r * src_pitch + c0 / 2 + seg * 8);
            const uint32_t w[2] = {v.x, v.y};
            uint32_t* trow = reinterpret_cast<uint32_t*>(&tile[row][seg * 16]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // 8 nibbles -> 8 bytes: even nibbles and odd nibbles separated, then interleaved byte-wise
                const uint32_t lo = w[h] & 0x0F0F0F0Fu, hi = (w[h] >> 4) & 0x0F0F0F0Fu;
                trow[2 * h] = __byte_perm(lo, hi, 0x5140);      // e0 e1 e2 e3
                trow[2 * h + 1] = __byte_perm(lo, hi, 0x7362);  // e4 e5 e6 e7
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int64_t c = c0 + seg * 16 + 2 * j;
                uint8_t v = 0;
                if (r < R && c < C) v = s[r * src_pitch + c / 2];
                tile[row][seg * 16 + 2 * j] = v & 0xF;
                tile[row][seg * 16 + 2 * j + 1] = (c + 1 < C) ? (v >> 4) : 0;
            }
        }
    }
    __syncthreads();
    {
        const int crow = t >> 2, seg = t & 3;  // 8 destination bytes = 16 elements of one destination row
        const int64_t c = c0 + crow;
        if (whole) {
            uint32_t o[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j)
                o[j >> 2] |= (uint32_t)(tile[seg * 16 + 2 * j][crow] | (tile[seg * 16 + 2 * j + 1][crow] << 4)) << (8 * (j & 3));
            *reinterpret_cast<uint2*>(d + c * dst_pitch + r0 / 2 + seg * 8) = make_uint2(o[0], o[1]);
        } else if (c < C) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int64_t r = r0 + seg * 16 + 2 * j;
                if (r < R) d[c * dst_pitch + r / 2] = (uint8_t)(tile[seg * 16 + 2 * j][crow] | (tile[seg * 16 + 2 * j + 1][crow] << 4));
            }
        }
    }
}

// The same rewrite for operands made of whole 64 x 128 tiles (R a multiple of 64, C of 128, 16-byte aligned source rows):
// 16-byte loads, nibbles widened to bytes into shared memory (pitch 33 words: conflict-free stores), then every thread
// takes an 8-row x 4-column block as eight words, transposes its bytes with byte permutes, packs each column's eight
// rows into one word and stores it; eight neighbouring lanes fill one 32-byte sector of a destination row.
__global__ void __launch_bounds__(256) fp4_transpose_tiles_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t src_pitch,
                                                                  int64_t dst_pitch, int64_t src_bs, int64_t dst_bs)
{
    __shared__ uint32_t tile[64][33];  // [source row][4 source columns per word, one element per byte]
    const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 128;
    const uint8_t* s = src + (int64_t)blockIdx.z * src_bs;
    uint8_t* d = dst + (int64_t)blockIdx.z * dst_bs;
    const int t = threadIdx.x;
    {
        const int row = t >> 2, seg = t & 3;  // 16 source bytes = 32 elements of one row
        const uint4 v = *reinterpret_cast<const uint4*>(s + (r0 + row) * src_pitch + c0 / 2 + seg * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const uint32_t lo = w[h] & 0x0F0F0F0Fu, hi = (w[h] >> 4) & 0x0F0F0F0Fu;
            tile[row][seg * 8 + 2 * h] = __byte_perm(lo, hi, 0x5140);      // e0 e1 e2 e3
            tile[row][seg * 8 + 2 * h + 1] = __byte_perm(lo, hi, 0x7362);  // e4 e5 e6 e7
        }
    }
    __syncthreads();
    const int r8 = t & 7, c4 = t >> 3;
    uint32_t a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = tile[r8 * 8 + i][c4];
    uint32_t o[4];
    {
        const uint32_t p0 = __byte_perm(a[0], a[1], 0x5140), p1 = __byte_perm(a[2], a[3], 0x5140);
        const uint32_t p2 = __byte_perm(a[0], a[1], 0x7362), p3 = __byte_perm(a[2], a[3], 0x7362);
        const uint32_t q0 = __byte_perm(a[4], a[5], 0x5140), q1 = __byte_perm(a[6], a[7], 0x5140);
        const uint32_t q2 = __byte_perm(a[4], a[5], 0x7362), q3 = __byte_perm(a[6], a[7], 0x7362);
        const uint32_t lo[4] = {__byte_perm(p0, p1, 0x5410), __byte_perm(p0, p1, 0x7632), __byte_perm(p2, p3, 0x5410), __byte_perm(p2, p3, 0x7632)};
        const uint32_t hi[4] = {__byte_perm(q0, q1, 0x5410), __byte_perm(q0, q1, 0x7632), __byte_perm(q2, q3, 0x5410), __byte_perm(q2, q3, 0x7632)};
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // bytes (rows 0..3), (rows 4..7) of column j -> eight nibbles, row 0 lowest
            const uint32_t y0 = lo[j] | (lo[j] >> 4), y1 = hi[j] | (hi[j] >> 4);
            o[j] = __byte_perm(y0, y1, 0x6420);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint32_t*>(d + (c0 + c4 * 4 + j) * dst_pitch + r0 / 2 + r8 * 4) = o[j];
}

// (R, C) fp4 packed along C -> (C, R) packed along R, for nb matrices; whole-tile operands take the word-wise kernel.
inline void fp4_transpose(const uint8_t* src, uint8_t* dst, int64_t R, int64_t C, int64_t src_pitch, int64_t dst_pitch, int64_t src_bs,
                          int64_t dst_bs, int64_t nb, cudaStream_t stream)
{
    const bool whole = R % 64 == 0 && C % 128 == 0 && src_pitch % 16 == 0 && src_bs % 16 == 0 && dst_pitch % 4 == 0 && dst_bs % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0 &&
                       getenv("OPSNN_FP4_TRANSPOSE_SIMPLE") == nullptr;
    if (whole)
        fp4_transpose_tiles_kernel<<<dim3((unsigned)(C / 128), (unsigned)(R / 64), (unsigned)nb), 256, 0, stream>>>(src, dst, src_pitch, dst_pitch,
                                                                                                                   src_bs, dst_bs);
    else
        fp4_transpose_kernel<<<dim3((unsigned)((C + 63) / 64), (unsigned)((R + 63) / 64), (unsigned)nb), 256, 0, stream>>>(src, dst, R, C, src_pitch,
                                                                                                                         dst_pitch, src_bs, dst_bs);
}

// 8-bit operand stored along n (x2 given as (k,n)) -> k-contiguous (n, kp) in workspace, kp = k rounded up to 16. The
// tensor core accepts the n-contiguous form, but with 224-column tiles the matmul kernel runs ~20 % slower on it (a CTA's
// 112-column share starts off the 32-byte sector grid); when one weight copy serves thousands of output rows, moving it
// once (2 bytes of traffic per element) costs a fraction of that.
// Tile = 64 k x 256 n bytes; 4 x 4 byte blocks are transposed in registers with byte permutes, 16-byte loads and stores.
__global__ void __launch_bounds__(256) byte_transpose_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t R, int64_t C,
                                                             int64_t src_pitch, int64_t dst_pitch, int64_t src_bs, int64_t dst_bs)
{
    __shared__ uint32_t tile[64][65];
    const int64_t r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 256;
    const uint8_t* s = src + (int64_t)blockIdx.z * src_bs;
    uint8_t* d = dst + (int64_t)blockIdx.z * dst_bs;
    const int t = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = i * 16 + (t >> 4), c16 = t & 15;
        const int64_t r = r0 + row, c = c0 + c16 * 16;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < R) {
            if (c + 16 <= C) {
                v = *reinterpret_cast<const uint4*>(s + r * src_pitch + c);
            } else if (c < C) {
                uint32_t w[4] = {0u, 0u, 0u, 0u};
                for (int j = 0; j < 16 && c + j < C; ++j) w[j >> 2] |= (uint32_t)s[r * src_pitch + c + j] << (8 * (j & 3));
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        tile[row][c16 * 4 + 0] = v.x; tile[row][c16 * 4 + 1] = v.y; tile[row][c16 * 4 + 2] = v.z; tile[row][c16 * 4 + 3] = v.w;
    }
    __syncthreads();
    const int k16 = t & 3, c4 = t >> 2;  // 16 source rows x 4 source columns -> 4 destination rows x 16 bytes
    uint32_t o[4][4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t a0 = tile[k16 * 16 + 4 * g + 0][c4], a1 = tile[k16 * 16 + 4 * g + 1][c4];
        const uint32_t a2 = tile[k16 * 16 + 4 * g + 2][c4], a3 = tile[k16 * 16 + 4 * g + 3][c4];
        const uint32_t t0 = __byte_perm(a0, a1, 0x5140), t1 = __byte_perm(a2, a3, 0x5140);
        const uint32_t t2 = __byte_perm(a0, a1, 0x7362), t3 = __byte_perm(a2, a3, 0x7362);
        o[0][g] = __byte_perm(t0, t1, 0x5410); o[1][g] = __byte_perm(t0, t1, 0x7632);
        o[2][g] = __byte_perm(t2, t3, 0x5410); o[3][g] = __byte_perm(t2, t3, 0x7632);
    }
    const int64_t kk = r0 + k16 * 16;
    if (kk < dst_pitch) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t c = c0 + c4 * 4 + j;
            if (c < C) *reinterpret_cast<uint4*>(d + c * dst_pitch + kk) = make_uint4(o[j][0], o[j][1], o[j][2], o[j][3]);
        }
    }
}

template <int BN, bool kF4>
__global__ void __launch_bounds__(192, 1)
qmm_mx_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const UmmaArgs a)
{
    constexpr int EW = 4;
    constexpr int kAtoms = kF4 ? 2 : 1;  // k atoms per stage: a stage is 128 bytes of k = 4 (fp8) / 8 (fp4) k-blocks of 32
    constexpr int RA = MxTile<BN>::kRowAtoms;
    constexpr uint32_t kSfaBytes = kAtoms * 512, kSfbBytes = kAtoms * RA * 512;
    constexpr uint32_t kBTile = MxTile<BN>::kBSmem;
    constexpr uint32_t kStage = kATile + kBTile + kSfaBytes + kSfbBytes;
    constexpr uint32_t kMxSfaCol = MxTile<BN>::kSfaCol;
    constexpr uint32_t kSfbCol = kMxSfaCol + 4 * kAtoms;
    constexpr uint32_t kAcc1 = MxTile<BN>::kAcc1Col;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * kStage);
    uint64_t* full = bars;
    uint64_t* empty = bars + a.stages;
    uint64_t* tfull = bars + 2 * a.stages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile uint32_t* abort_flag = tmem_ptr + 1;
    float* s_bias = reinterpret_cast<float*>(tmem_ptr + 4);  // [256]

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&tfull[b], 1);
            ptx::mbar_init(&tempty[b], EW);  // one arrival per epilogue warp
        }
        *abort_flag = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == EW + 1) ptx::tmem_alloc(tmem_ptr, kTmemCols);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    const uint32_t tiles_per_batch = (uint32_t)a.tiles_m * (uint32_t)a.tiles_n;
    const uint32_t ntiles = (uint32_t)a.num_tiles;
    const uint32_t smem0 = ptx::smem_u32(smem), full0 = ptx::smem_u32(full), empty0 = ptx::smem_u32(empty);
    const uint32_t stages = (uint32_t)a.stages;
    const int kstages = a.kblocks;  // 128-byte k stages per tile

    if (warp == EW) {
        // ======================= producer: two TMA loads and two scale-atom bulk copies per stage =======================
        if (lane == 0) {
            ptx::tma_prefetch_desc(&map_a);
            ptx::tma_prefetch_desc(&map_b);
        }
        __syncwarp();
        uint32_t s = 0, par = 0;
        bool ok = true;
        const bool b_mn = a.b_mn_major != 0, a_mn = a.a_mn_major != 0;
        for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<16>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int32_t m0 = (int32_t)tm * BM, n0 = (int32_t)tn * BN;
            const int32_t ba = a.a_batched ? (int32_t)b : 0, bb = a.b_batched ? (int32_t)b : 0;
            const uint8_t* sfa = a.sfa + (int64_t)ba * a.sfa_bs + ((int64_t)tm * kstages) * kSfaBytes;
            const uint8_t* sfb = a.sfb + (int64_t)bb * a.sfb_bs + ((int64_t)tn * kstages) * kSfbBytes;
            // bytes one stage's copies deliver: k-major B is one box of BN rows, n-major B whole 128-column boxes
            const uint32_t tx = (uint32_t)kATile + (b_mn ? kBTile : (uint32_t)(BN * BK)) + kSfaBytes + kSfbBytes;
            int32_t kk = 0;
            for (int kb = 0; kb < kstages; ++kb) {
                if (!ptx::mbar_wait_a(empty0 + 8u * s, par ^ 1u, abort_flag)) {
                    report(abort_flag, (1u << 8) | 1u);
                    ok = false;
                    break;
                }
                if (ptx::elect_one()) {
                    const uint32_t fb = full0 + 8u * s, sa = smem0 + s * kStage, sb = sa + (uint32_t)kATile;
                    ptx::mbar_expect_tx_a(fb, tx);
                    ptx::tma_load_3d_a(sa, &map_a, fb, a_mn ? m0 : kk, a_mn ? kk : m0, ba);
                    ptx::tma_load_3d_a(sb, &map_b, fb, b_mn ? n0 : kk, b_mn ? kk : n0, bb);
                    if (BN > 128 && b_mn) ptx::tma_load_3d_a(sb + 128u * BK, &map_b, fb, n0 + 128, kk, bb);
                    ptx::bulk_load_a(sb + kBTile, sfa, kSfaBytes, fb);
                    ptx::bulk_load_a(sb + kBTile + kSfaBytes, sfb, kSfbBytes, fb);
                }
                __syncwarp();
                sfa += kSfaBytes;
                sfb += kSfbBytes;
                kk += BK;
                if (++s == stages) {
                    s = 0;
                    par ^= 1u;
                }
            }
        }
    } else if (warp == EW + 1) {
        // ======================= MMA issuer =======================
        uint32_t s = 0, par = 0, grp = 0;
        bool ok = true;
        const uint32_t tfull0 = ptx::smem_u32(tfull), tempty0 = ptx::smem_u32(tempty);
        const uint64_t da0 = a.a_mn_major ? ptx::make_smem_desc(smem0, 128 * BK, 1024, 2) : ptx::make_smem_desc(smem0, 0, 1024, 2);
        const uint64_t db0 = a.b_mn_major ? ptx::make_smem_desc(smem0 + kATile, 128 * BK, 1024, 2)
                                          : ptx::make_smem_desc(smem0 + kATile, 0, 1024, 2);
        const uint64_t dsf0 = ptx::make_smem_desc(smem0 + kATile + kBTile, 0, 128, 0);  // 32 rows x 16 bytes, no swizzle
        const uint32_t a_lo = (uint32_t)da0, b_lo = (uint32_t)db0, sf_lo = (uint32_t)dsf0;
        const uint64_t a_hi = da0 & 0xFFFFFFFF00000000ull, b_hi = db0 & 0xFFFFFFFF00000000ull, sf_hi = dsf0 & 0xFFFFFFFF00000000ull;
        const uint32_t a_k1 = a.a_mn_major ? 256u : 2u, b_k1 = a.b_mn_major ? 256u : 2u;
        const uint32_t idesc = a.idesc;
        for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            uint32_t acc = 0u;
            if (!ptx::mbar_wait_a(tempty0 + 8u * (grp & 1u), ((grp >> 1) & 1u) ^ 1u, abort_flag)) {
                report(abort_flag, (2u << 8) | 1u);
                ok = false;
                break;
            }
            for (int kb = 0; kb < kstages; ++kb) {
                if (!ptx::mbar_wait_a(full0 + 8u * s, par, abort_flag)) {
                    report(abort_flag, (2u << 8) | 2u);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (ptx::elect_one()) {
                    const uint32_t stage_off = (s * kStage) >> 4;
                    const uint32_t d = tmem_base + (grp & 1u) * kAcc1;
                    const uint32_t al = a_lo + stage_off, bl = b_lo + stage_off, sl = sf_lo + stage_off;
                    // scale atoms shared -> TMEM: A's k atoms, then B's (k atom, row atom) pairs, in shared-memory order
#pragma unroll
                    for (int at = 0; at < kAtoms; ++at) ptx::tmem_cp_sf(tmem_base + kMxSfaCol + 4 * at, sf_hi | (uint64_t)(sl + at * 32));
#pragma unroll
                    for (int at = 0; at < kAtoms * RA; ++at)
                        ptx::tmem_cp_sf(tmem_base + kSfbCol + 4 * at, sf_hi | (uint64_t)(sl + (kAtoms + at) * 32));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t sf_id = kF4 ? (uint32_t)(k & 1) * 2u : (uint32_t)k;
                        const uint32_t katom = kF4 ? (uint32_t)(k >> 1) : 0u;
                        const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                        const uint64_t da = a_hi | (uint64_t)(al + k * a_k1), db = b_hi | (uint64_t)(bl + k * b_k1);
                        const uint32_t ta = tmem_base + kMxSfaCol + 4u * katom, tb = tmem_base + kSfbCol + 4u * RA * katom;
                        if (kF4) ptx::umma_mxf4(d, da, db, id, ta, tb, k == 0 ? acc : 1u);
                        else ptx::umma_mxf8f6f4(d, da, db, id, ta, tb, k == 0 ? acc : 1u);
                    }
                    ptx::umma_commit_a(empty0 + 8u * s);
                }
                __syncwarp();
                acc = 1u;
                if (++s == stages) {
                    s = 0;
                    par ^= 1u;
                }
            }
            if (ok) {
                if (ptx::elect_one()) ptx::umma_commit_a(tfull0 + 8u * (grp & 1u));
                __syncwarp();
                ++grp;
            }
        }
    } else {
        // ======================= epilogue warps: acc (+ bias) -> output dtype =======================
        const int quad = warp & 3;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        uint32_t grp = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<16>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
            const int64_t row = m0 + quad * 32 + lane;
            const bool row_ok = row < a.m;
            const int out_bytes = a.out_dtype == ACL_FLOAT ? 4 : 2;
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + b * a.out_bs * out_bytes;
            const uint32_t buf = grp & 1, gpar = (grp >> 1) & 1;
            const uint8_t* bias = reinterpret_cast<const uint8_t*>(a.bias);
            if (bias != nullptr) bias += b * a.bias_bs * (a.bias_dtype == ACL_FLOAT ? 4 : 2);
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's readers of s_bias are done
            for (int c = threadIdx.x; c < BN; c += 128)
                s_bias[c] = bias != nullptr ? load_as_float(bias, min(n0 + c, a.n - 1), a.bias_dtype) : 0.f;
            if (!ptx::mbar_wait_relaxed(&tfull[buf], gpar, abort_flag)) report(abort_flag, (3u << 8) | 1u);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*abort_flag != 0u) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                ptx::tmem_ld32(tmem_base + lane_addr + buf * kAcc1 + c, v);
                ptx::tmem_ld_wait();
                const int64_t col = n0 + c;
                const int valid = (int)min((int64_t)32, a.n - col);
                if (row_ok && valid > 0) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(s_bias + c + i);
                        f[i] = __fadd_rn(__uint_as_float(v[i]), b4.x);
                        f[i + 1] = __fadd_rn(__uint_as_float(v[i + 1]), b4.y);
                        f[i + 2] = __fadd_rn(__uint_as_float(v[i + 2]), b4.z);
                        f[i + 3] = __fadd_rn(__uint_as_float(v[i + 3]), b4.w);
                    }
                    store_row32(a, out, row, col, f, valid);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&tempty[buf]);
            ++grp;
        }
    }
    if (*abort_flag != 0u) __nanosleep(200000);  // lets copies that are still in flight land before the CTA leaves
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == EW + 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

bool is_fp4(int dt) { return dt == ACL_FLOAT4_E2M1; }

template <bool kF4>
int32_t mx_launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream);  // qmm_mx_umma_pair.cuh

struct MxPlan {
    bool f4, pair;
    int bn, atoms, row_atoms;
    int64_t tiles_m, tiles_n, kstages, kblocks32, kq;
    uint64_t sfa_bytes_per_batch, sfb_bytes_per_batch, nb_a, nb_b;
    bool tr_a, tr_b;               // operand stored along m / n rewritten k-contiguous into workspace first: always for fp4,
                                   // for an 8-bit x2 when one copy of it serves enough output rows to pay for the move
    uint64_t tr_a_bytes, tr_b_bytes;  // whole operand, all batches
};

// Host tile selection: 224-column tiles (less operand traffic per flop) whenever they still give every SM a tile.
int mx_pick_bn(const OpsnnQmmParams* p)
{
    if (const char* e = getenv("OPSNN_QMM_MX_BN")) {
        const int v = atoi(e);
        if (v == 128 || v == 224) return v;
    }
    if (p->n <= 128) return 128;
    const int64_t tiles = p->batch * ((p->m + BM - 1) / BM) * ((p->n + 223) / 224);
    return tiles >= 148 ? 224 : 128;
}

// The x2 the matmul kernel will see when the caller handed over a prepared k-contiguous copy.
OpsnnQmmParams mx_effective(const OpsnnQmmParams* p)
{
    OpsnnQmmParams e = *p;
    if (p->prep_b != nullptr) {
        e.b = p->prep_b;
        e.b_ld = p->k;
        e.b_bs = p->b_bs != 0 ? p->n * p->k : 0;
        e.trans_b = 1;
    }
    return e;
}

MxPlan mx_plan(const OpsnnQmmParams* p)
{
    MxPlan q{};
    q.f4 = is_fp4(p->a_dtype);
    q.bn = mx_pick_bn(p);
    q.atoms = q.f4 ? 2 : 1;
    q.row_atoms = q.bn > 128 ? 2 : 1;
    const int64_t k_per_stage = q.f4 ? 256 : 128;
    q.tiles_m = (p->m + BM - 1) / BM;  // 128-row tiles: the unit of A's scale atoms, also when CTA pairs share 256-row tiles
    q.tiles_n = (p->n + q.bn - 1) / q.bn;
    // CTA pairs (256 x 224 tiles, each CTA loading half of B) when there is a tile for about every pair of SMs
    q.pair = q.bn == 224 && p->m >= 256 && p->batch * ((p->m + 255) / 256) * q.tiles_n >= 74;
    if (const char* e = getenv("OPSNN_QMM_PAIR")) q.pair = atoi(e) != 0 && q.bn == 224;
    q.kstages = (p->k + k_per_stage - 1) / k_per_stage;
    q.kblocks32 = (p->k + 31) / 32;
    q.kq = (p->k + 63) / 64;
    q.nb_a = p->sa_bs != 0 ? (uint64_t)p->batch : 1;
    q.nb_b = p->sb_bs != 0 ? (uint64_t)p->batch : 1;
    q.tr_a = q.f4 && p->trans_a != 0;
    q.tr_b = q.f4 && p->trans_b == 0;
    if (!q.f4 && p->trans_b == 0 && getenv("OPSNN_MX_NO_TRANSPOSE") == nullptr)
        q.tr_b = q.bn == 224 && p->m * (p->b_bs == 0 ? p->batch : 1) >= 4096 && (p->b_bs == 0 || p->batch <= 65535) && p->k / 64 < 65535;
    q.tr_a_bytes = q.tr_a ? (uint64_t)(p->a_bs != 0 ? p->batch : 1) * (uint64_t)p->m * (uint64_t)(p->k / 2) : 0;
    q.tr_b_bytes = q.tr_b ? (uint64_t)(p->b_bs != 0 ? p->batch : 1) * (uint64_t)p->n * (uint64_t)(q.f4 ? p->k / 2 : p->k) : 0;
    q.sfa_bytes_per_batch = (uint64_t)q.tiles_m * q.kstages * q.atoms * 512;
    q.sfb_bytes_per_batch = (uint64_t)q.tiles_n * q.kstages * q.atoms * q.row_atoms * 512;
    return q;
}

template <int BN, bool kF4>
int32_t mx_launch_one(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    constexpr uint32_t stage = (uint32_t)kATile + MxTile<BN>::kBSmem + (kF4 ? 2 : 1) * 512 * (1 + MxTile<BN>::kRowAtoms);
    int stages = (227 * 1024 - 2048) / (int)stage;
    if (stages > 8) stages = 8;
    if (stages > a.kblocks + 1) stages = a.kblocks + 1 > 2 ? a.kblocks + 1 : 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * stage + 1024 + 256 + 256 * 4;
    const int64_t grid = a.num_tiles < sm_count() ? a.num_tiles : sm_count();
    static std::atomic<uint64_t> configured{0};
    {
        const cudaError_t rc = once_per_device(
            configured, [&] { return cudaFuncSetAttribute(qmm_mx_umma_kernel<BN, kF4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); });
        if (rc != cudaSuccess) return (int32_t)rc;
    }
    qmm_mx_umma_kernel<BN, kF4><<<(unsigned)grid, 192, smem, stream>>>(ma, mb, a);
    note_launch(kF4 ? "qmm_umma_mxfp4" : "qmm_umma_mxfp8");
    return (int32_t)cudaGetLastError();
}

}  // namespace

bool qmm_mx_umma_eligible(const OpsnnQmmParams* p)
{
    if (p->mode != OPSNN_QMM_MX) return false;
    const bool f8 = is_fp8(p->a_dtype) && is_fp8(p->b_dtype);
    const bool f4 = is_fp4(p->a_dtype) && is_fp4(p->b_dtype);
    if (!f8 && !f4) return false;
    if (p->scale_b_dtype != ACL_FLOAT8_E8M0 || p->scale_a == nullptr || p->scale_b == nullptr) return false;
    if (p->group_k != 32 || p->k % 32 != 0) return false;
    if (p->out_dtype != ACL_BF16 && p->out_dtype != ACL_FLOAT16 && p->out_dtype != ACL_FLOAT) return false;
    if (p->bias != nullptr && p->bias_dtype != ACL_FLOAT && p->bias_dtype != ACL_BF16 && p->bias_dtype != ACL_FLOAT16) return false;
    const int64_t div = f4 ? 2 : 1;  // elements per byte
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al16(p->a) || !al16(p->b)) return false;
    if ((p->a_ld / div) % 16 != 0 || (p->b_ld / div) % 16 != 0 || (p->a_bs / div) % 16 != 0 || (p->b_bs / div) % 16 != 0) return false;
    if (f4 && (p->a_ld % 2 != 0 || p->b_ld % 2 != 0 || p->a_bs % 2 != 0 || p->b_bs % 2 != 0)) return false;
    if (p->m < 1 || p->n < 1 || p->k < 1 || p->batch < 1 || p->batch > 0x7FFFFFFF) return false;
    if (p->batch * ((p->m + 127) / 128) * ((p->n + 127) / 128) > 0x7FFFFFFF) return false;
    if (p->m > 0x7FFFFF00 || p->n > 0x7FFFFF00 || p->k > 0x7FFFFF00) return false;
    return true;
}

uint64_t qmm_mx_umma_workspace_size(const OpsnnQmmParams* p0)
{
    const OpsnnQmmParams pe = mx_effective(p0);
    const OpsnnQmmParams* p = &pe;
    const MxPlan q = mx_plan(p);
    return q.nb_a * q.sfa_bytes_per_batch + q.nb_b * q.sfb_bytes_per_batch + q.tr_a_bytes + q.tr_b_bytes + 3 * 256;
}

// x2Scale of p (all batches) into scale-atom order at dst, for the tile width of plan q.
static void mx_relayout_sfb(const OpsnnQmmParams* p, const MxPlan& q, int scale_b_k_major, uint8_t* dst, cudaStream_t stream)
{
    const int64_t gb = (int64_t)q.nb_b * q.tiles_n * q.row_atoms;
    if (getenv("OPSNN_MX_SF_SIMPLE") == nullptr && gb < 0x7FFFFFFF) {
        mx_sf_relayout_tiled_kernel<<<(unsigned)gb, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(p->scale_b), dst, p->n, q.kblocks32, q.kq,
                                                                      scale_b_k_major, q.tiles_n, q.kstages, q.atoms, p->sb_bs, q.bn, q.row_atoms);
    } else {
        const int64_t wb = (int64_t)q.nb_b * q.tiles_n * q.kstages * q.atoms * q.row_atoms * 128;
        mx_sf_relayout_kernel<<<(unsigned)std::min<int64_t>((wb + 255) / 256, 148 * 16), 256, 0, stream>>>(
            reinterpret_cast<const uint8_t*>(p->scale_b), dst, p->n, q.kblocks32, q.kq, scale_b_k_major, q.tiles_n, q.kstages, q.atoms,
            (int64_t)q.nb_b, p->sb_bs, q.bn, q.row_atoms);
    }
}

// x2 stored (k, n) (all batches) rewritten (n, k) at dst.
static void mx_transpose_b(const OpsnnQmmParams* p, bool f4, uint8_t* dst, cudaStream_t stream)
{
    const int64_t nb = p->b_bs != 0 ? p->batch : 1;
    if (f4) {
        fp4_transpose(reinterpret_cast<const uint8_t*>(p->b), dst, p->k, p->n, p->b_ld / 2, p->k / 2, p->b_bs / 2, p->n * (p->k / 2), nb, stream);
        note_launch("fp4_transpose");
    } else {
        byte_transpose_kernel<<<dim3((unsigned)((p->n + 255) / 256), (unsigned)((p->k + 63) / 64), (unsigned)nb), 256, 0, stream>>>(
            reinterpret_cast<const uint8_t*>(p->b), dst, p->k, p->n, p->b_ld, p->k, p->b_bs, p->n * p->k);
        note_launch("byte_transpose");
    }
}

uint64_t qmm_mx_prepare_b_size(const OpsnnQmmParams* p)
{
    if (!qmm_mx_umma_eligible(p)) return 0;
    const MxPlan q = mx_plan(p);
    const bool move = p->trans_b == 0 && (q.f4 || (p->k % 32 == 0 && p->k / 64 < 65535 && (p->b_bs == 0 || p->batch <= 65535)));
    const uint64_t copy = move ? (uint64_t)(p->b_bs != 0 ? p->batch : 1) * (uint64_t)p->n * (uint64_t)(q.f4 ? p->k / 2 : p->k) : 0;
    return ((q.nb_b * q.sfb_bytes_per_batch + 255) & ~(uint64_t)255) + copy + 256;
}

int32_t qmm_mx_prepare_b_launch(const OpsnnQmmParams* p, void* storage, uint64_t storage_size, const void** prep_b, const void** prep_sfb,
                                int32_t* prep_bn, cudaStream_t stream)
{
    *prep_b = *prep_sfb = nullptr;
    *prep_bn = 0;
    if (!qmm_mx_umma_eligible(p) || p->prep_b != nullptr || p->prep_sfb != nullptr) return 0;
    const uint64_t need = qmm_mx_prepare_b_size(p);
    if (storage == nullptr || storage_size < need) return (int32_t)cudaErrorInvalidValue;
    const MxPlan q = mx_plan(p);
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(storage) + 255) & ~(uintptr_t)255);
    mx_relayout_sfb(p, q, p->trans_b ? 0 : 1, base, stream);
    note_launch("mx_sf_relayout", 1);
    *prep_sfb = base;
    *prep_bn = q.bn;
    const bool move = p->trans_b == 0 && (q.f4 || (p->k % 32 == 0 && p->k / 64 < 65535 && (p->b_bs == 0 || p->batch <= 65535)));
    if (move) {
        uint8_t* copy = base + ((q.nb_b * q.sfb_bytes_per_batch + 255) & ~(uint64_t)255);
        mx_transpose_b(p, q.f4, copy, stream);
        *prep_b = copy;
    }
    return (int32_t)cudaGetLastError();
}

int32_t qmm_mx_umma_launch(const OpsnnQmmParams* p0, cudaStream_t stream)
{
    const OpsnnQmmParams pe = mx_effective(p0);  // a prepared k-contiguous copy of x2 replaces the caller's (k,n) one
    const OpsnnQmmParams* p = &pe;
    const MxPlan q = mx_plan(p);
    if (p->workspace == nullptr || p->workspace_size < qmm_mx_umma_workspace_size(p0)) return (int32_t)cudaErrorInvalidValue;
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p->workspace) + 255) & ~(uintptr_t)255);
    uint8_t* sfa = ws;
    uint8_t* sfb = ws + q.nb_a * q.sfa_bytes_per_batch;
    // x2Scale keeps the caller's storage order even when x2 itself was moved: (kq, n, 2) for x2 given as (k,n), (n, kq, 2) for (n,k)
    const int scale_b_k_major = p0->trans_b ? 0 : 1;
    const bool sfb_ready = p0->prep_sfb != nullptr && p0->prep_bn == q.bn;
    // ---- pre-pass: both operands' scales into atom order ----
    {
        const int64_t wa = (int64_t)q.nb_a * q.tiles_m * q.kstages * q.atoms * 128;
        const int64_t wb = (int64_t)q.nb_b * q.tiles_n * q.kstages * q.atoms * q.row_atoms * 128;
        const int threads = 256;
        const auto blocks = [&](int64_t w) { return (unsigned)std::min<int64_t>((w + threads - 1) / threads, 148 * 16); };
        // x1Scale is (m, kq, 2), or (kq, m, 2) when x1 is stored (k,m); x2Scale is (kq, n, 2), or (n, kq, 2) when x2 is stored (n,k)
        const int64_t ga = (int64_t)q.nb_a * q.tiles_m, gb = (int64_t)q.nb_b * q.tiles_n * q.row_atoms;
        (void)wb;
        (void)gb;
        if (getenv("OPSNN_MX_SF_SIMPLE") == nullptr && ga < 0x7FFFFFFF) {
            mx_sf_relayout_tiled_kernel<<<(unsigned)ga, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(p->scale_a), sfa, p->m, q.kblocks32,
                                                                          q.kq, p->trans_a ? 1 : 0, q.tiles_m, q.kstages, q.atoms, p->sa_bs, BM, 1);
        } else {
            mx_sf_relayout_kernel<<<blocks(wa), threads, 0, stream>>>(reinterpret_cast<const uint8_t*>(p->scale_a), sfa, p->m, q.kblocks32, q.kq,
                                                                      p->trans_a ? 1 : 0, q.tiles_m, q.kstages, q.atoms, (int64_t)q.nb_a, p->sa_bs,
                                                                      BM, 1);
        }
        if (sfb_ready) sfb = const_cast<uint8_t*>(static_cast<const uint8_t*>(p0->prep_sfb));
        else mx_relayout_sfb(p, q, scale_b_k_major, sfb, stream);
        note_launch("mx_sf_relayout", sfb_ready ? 1 : 2);
    }
    // ---- pre-pass: fp4 operands that are not k-contiguous ----
    OpsnnQmmParams pk = *p;  // the operand views the matmul kernel sees
    {
        auto up = [](uint8_t* x) { return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(x) + 255) & ~(uintptr_t)255); };
        uint8_t* next = up(ws + q.nb_a * q.sfa_bytes_per_batch + q.nb_b * q.sfb_bytes_per_batch);
        if (q.tr_a) {  // stored (k, m) -> (m, k)
            const int64_t nb = p->a_bs != 0 ? p->batch : 1;
            fp4_transpose(reinterpret_cast<const uint8_t*>(p->a), next, p->k, p->m, p->a_ld / 2, p->k / 2, p->a_bs / 2, p->m * (p->k / 2), nb, stream);
            pk.a = next; pk.a_ld = p->k; pk.a_bs = p->a_bs != 0 ? p->m * p->k : 0; pk.trans_a = 0;
            next = up(next + q.tr_a_bytes);
            note_launch("fp4_transpose");
        }
        if (q.tr_b && !q.f4) {  // 8-bit, stored (k, n) -> (n, k); k is a multiple of 32 here
            const int64_t nb = p->b_bs != 0 ? p->batch : 1;
            byte_transpose_kernel<<<dim3((unsigned)((p->n + 255) / 256), (unsigned)((p->k + 63) / 64), (unsigned)nb), 256, 0, stream>>>(
                reinterpret_cast<const uint8_t*>(p->b), next, p->k, p->n, p->b_ld, p->k, p->b_bs, p->n * p->k);
            pk.b = next; pk.b_ld = p->k; pk.b_bs = p->b_bs != 0 ? p->n * p->k : 0; pk.trans_b = 1;
            note_launch("byte_transpose");
        } else if (q.tr_b) {  // stored (k, n) -> (n, k)
            const int64_t nb = p->b_bs != 0 ? p->batch : 1;
            fp4_transpose(reinterpret_cast<const uint8_t*>(p->b), next, p->k, p->n, p->b_ld / 2, p->k / 2, p->b_bs / 2, p->n * (p->k / 2), nb, stream);
            pk.b = next; pk.b_ld = p->k; pk.b_bs = p->b_bs != 0 ? p->n * p->k : 0; pk.trans_b = 1;
            note_launch("fp4_transpose");
        }
    }
    const OpsnnQmmParams* po = p;  // original: scale layouts follow the caller's storage
    (void)po;
    p = &pk;
    UmmaArgs a{};
    a.mode = p->mode;
    a.a_mn_major = p->trans_a ? 1 : 0;
    a.b_mn_major = p->trans_b ? 0 : 1;
    a.batch = p->batch; a.m = p->m; a.n = p->n; a.k = p->k;
    a.tiles_m = q.pair ? (int32_t)((p->m + 255) / 256) : (int32_t)q.tiles_m;
    a.tiles_n = (int32_t)q.tiles_n;
    a.kblocks = (int32_t)q.kstages;
    a.num_tiles = p->batch * a.tiles_m * a.tiles_n;
    a.a_batched = p->a_bs != 0;
    a.b_batched = p->b_bs != 0;
    a.out_dtype = p->out_dtype; a.bias_dtype = p->bias_dtype;
    a.bias = p->bias; a.bias_bs = p->bias_bs; a.out = p->out; a.out_ld = p->out_ld; a.out_bs = p->out_bs;
    a.sfa = sfa; a.sfb = sfb;
    a.sfa_bs = q.nb_a > 1 ? (int64_t)q.sfa_bytes_per_batch : 0;
    a.sfb_bs = q.nb_b > 1 ? (int64_t)q.sfb_bytes_per_batch : 0;
    const uint32_t fa = q.f4 ? 1u : (p->a_dtype == ACL_FLOAT8_E5M2 ? 1u : 0u);
    const uint32_t fb = q.f4 ? 1u : (p->b_dtype == ACL_FLOAT8_E5M2 ? 1u : 0u);
    a.idesc = make_idesc_block_scaled(fa, fb, (uint32_t)a.a_mn_major, (uint32_t)a.b_mn_major, q.pair ? 256u : (uint32_t)BM, (uint32_t)q.bn);

    const uint64_t div = q.f4 ? 2 : 1;
    CUtensorMap ma, mb;
    const uint64_t nb_a = a.a_batched ? (uint64_t)p->batch : 1, nb_b = a.b_batched ? (uint64_t)p->batch : 1;
    bool ok;
    if (a.a_mn_major) ok = make_map(&ma, p->a, (uint64_t)p->m, (uint64_t)p->k, nb_a, (uint64_t)p->a_ld, (uint64_t)p->a_bs, 128);
    else ok = make_map(&ma, p->a, (uint64_t)p->k / div, (uint64_t)p->m, nb_a, (uint64_t)p->a_ld / div, (uint64_t)p->a_bs / div, 128);
    if (a.b_mn_major) ok = ok && make_map(&mb, p->b, (uint64_t)p->n, (uint64_t)p->k, nb_b, (uint64_t)p->b_ld, (uint64_t)p->b_bs, 128);
    else ok = ok && make_map(&mb, p->b, (uint64_t)p->k / div, (uint64_t)p->n, nb_b, (uint64_t)p->b_ld / div, (uint64_t)p->b_bs / div, q.pair ? 112u : (uint32_t)q.bn);
    if (!ok) return (int32_t)cudaErrorInvalidValue;

    if (q.pair) return q.f4 ? mx_launch_pair<true>(ma, mb, a, stream) : mx_launch_pair<false>(ma, mb, a, stream);
    if (q.bn == 224) return q.f4 ? mx_launch_one<224, true>(ma, mb, a, stream) : mx_launch_one<224, false>(ma, mb, a, stream);
    return q.f4 ? mx_launch_one<128, true>(ma, mb, a, stream) : mx_launch_one<128, false>(ma, mb, a, stream);
}
