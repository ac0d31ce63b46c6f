// rank1_gemm: M[e,i,j] (op)= sum_q W[e,q] * B1[q,i] * B2[q,j]   (element mass-matrix assembly).
//
// Viewed as one GEMM  M[e,(i,j)] = sum_q W[e,q] * BB[q,(i,j)],  BB[q,(i,j)] = B1[q,i]*B2[q,j]:
// E x 64 times 64 x (NI*NJ).  It is compute bound on fp64 (2*64*NI*NJ flops against
// 8*(64 + NI*NJ) bytes per element: 14.7 flop/byte for 27 x 27), so it runs on the fp64
// tensor cores (mma.sync m8n8k4).  A CTA owns 32 elements: their W rows arrive by
// asynchronous bulk copies into rows padded to 68 doubles (conflict-free fragment loads),
// double buffered; B1, B2 sit in shared memory for the whole kernel and the BB operand is
// formed on the fly (one multiply per fragment entry, reused by the four 8-element row
// tiles of the warp: 3 % extra fp64 work).  A warp computes 32 elements x 32 columns at a
// time (16 accumulator tiles), then routes each 8 x 32 block through a small per-warp
// staging area so that rows leave as contiguous 256-byte stores.
//
// When B1 and B2 are the same matrix, M_e is symmetric: a second kernel (further down)
// computes only the ni*(ni+1)/2 columns with i <= j and writes every off-diagonal entry
// twice, at (i,j) and (j,i), which halves the tensor-core work (the two products
// (W*B_i)*B_j and (W*B_j)*B_i differ only in rounding, well inside the tolerance).
// Measured on B200, E = 2^18, 27 x 27: general kernel 0.926 ms; symmetric columns with the
// mirrored entries stored straight to global memory 1.18 ms (scattered 8-byte stores);
// symmetric columns through a shared-memory image and one bulk store 0.583 ms.
//
// Algorithmic HBM traffic per element: 8*64 (W) + 8*NI*NJ (M) bytes.
#include "common.cuh"
#include "dmma.cuh"

#include <cstdlib>
#include "tma.cuh"
#include "tmem.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int QN = 64;                 // largest contracted extent
constexpr int ET = 32;                 // elements per CTA tile (4 row tiles of 8)
constexpr int LDW = QN + 4;            // padded W row
constexpr int NTHREADS = 256;
constexpr int WARPS = NTHREADS / 32;
constexpr int MAXN = 32;               // NI, NJ <= 32
constexpr int LDS_STAGE = 40;          // staging row (doubles)

struct Smem
{
    double W[2][ET * LDW];
    double B1[QN * MAXN];
    double B2[QN * MAXN];
    double stage[WARPS][8 * LDS_STAGE];
    uint64_t full[2];
};

struct Rank1Args
{
    const double *W;
    const double *B1;
    const double *B2;
    double *M;
    int64_t elements;
    int q;          // contracted extent, 1 .. QN
    int ni, nj;
    int op;
    int *wait_flag;
    int use_bulk;
};

__device__ __forceinline__ void issue_w_load(Smem &s, const Rank1Args &a, int64_t tile, int buf)
{
    const int64_t e0 = tile * ET;
    if (!a.use_bulk || e0 >= a.elements) return;
    if (threadIdx.x < 32)
    {
        const int64_t left = a.elements - e0;
        const int n_e = left < ET ? static_cast<int>(left) : ET;
        if (threadIdx.x == 0) mbar_arrive_expect_tx(&s.full[buf], n_e * a.q * 8);
        __syncwarp();
        if (static_cast<int>(threadIdx.x) < n_e)
            bulk_load(&s.W[buf][threadIdx.x * LDW], a.W + (e0 + threadIdx.x) * a.q, a.q * 8, &s.full[buf]);
    }
}

// NTG: 8-column tiles per column group of a warp.
template <int NTG>
__global__ void __launch_bounds__(NTHREADS, 2)
rank1_gemm_kernel(const Rank1Args a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    Smem &s = *reinterpret_cast<Smem *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ni = a.ni, nj = a.nj, nc = ni * nj;
    const int n_cols = nc;
    constexpr int GW = NTG * 8;                            // columns per group
    const int n_groups = (n_cols + GW - 1) / GW;
    const int64_t n_tiles = (a.elements + ET - 1) / ET;

    if (tid == 0)
    {
        mbar_init(&s.full[0], 1);
        mbar_init(&s.full[1], 1);
        fence_mbar_init();
    }
    // The contracted extent is processed in steps of four: rows q .. q4-1 of B1, B2 and the same
    // columns of every W row are zero, so that they add nothing.
    const int q4 = (a.q + 3) & ~3;
    for (int i = tid; i < q4 * ni; i += NTHREADS) s.B1[i] = i < a.q * ni ? a.B1[i] : 0.0;
    for (int i = tid; i < q4 * nj; i += NTHREADS) s.B2[i] = i < a.q * nj ? a.B2[i] : 0.0;
    for (int i = tid; i < 2 * ET * (q4 - a.q); i += NTHREADS)
        s.W[0][(i / (q4 - a.q)) * LDW + a.q + i % (q4 - a.q)] = 0.0;     // the two buffers are contiguous: rows 0 .. 2*ET-1
    __syncthreads();

    int64_t tile = blockIdx.x;
    issue_w_load(s, a, tile, 0);
    uint32_t phase_bits = 0;
    int buf = 0;
    double *stg = s.stage[warp];

    for (; tile < n_tiles; tile += gridDim.x)
    {
        issue_w_load(s, a, tile + gridDim.x, buf ^ 1);   // released by the barrier that closed the previous tile
        const int64_t e0 = tile * ET;
        const int64_t left = a.elements - e0;
        const int n_e = left < ET ? static_cast<int>(left) : ET;
        if (a.use_bulk)
        {
            if (!mbar_wait(&s.full[buf], (phase_bits >> buf) & 1u)) atomicExch(a.wait_flag, 1);
            phase_bits ^= (1u << buf);
        }
        else
        {
            for (int i = tid; i < n_e * a.q; i += NTHREADS) s.W[buf][(i / a.q) * LDW + (i % a.q)] = __ldcs(a.W + e0 * a.q + i);
            __syncthreads();
        }
        const double *sw = s.W[buf];

        for (int grp = warp; grp < n_groups; grp += WARPS)
        {
            const int c0 = grp * GW;
            // column -> (i, j) of this lane's B-fragment column in each column tile
            int off1[NTG], off2[NTG];
#pragma unroll
            for (int nt = 0; nt < NTG; ++nt)
            {
                int c = c0 + nt * 8 + g;
                c = c < n_cols ? c : n_cols - 1;   // padded columns compute a copy that is never stored
                off1[nt] = c / nj;
                off2[nt] = c - off1[nt] * nj;
            }
            double acc[4][NTG][2];
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTG; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = 0.0;

#pragma unroll 2
            for (int k0 = 0; k0 < q4; k0 += 4)
            {
                double af[4], bf[NTG];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) af[mt] = sw[(mt * 8 + g) * LDW + k0 + t];
                const double *b1 = s.B1 + (k0 + t) * ni;
                const double *b2 = s.B2 + (k0 + t) * nj;
#pragma unroll
                for (int nt = 0; nt < NTG; ++nt) bf[nt] = b1[off1[nt]] * b2[off2[nt]];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NTG; ++nt) dmma_m8n8k4(acc[mt][nt], af[mt], bf[nt]);
            }

            // epilogue: 8 x GW blocks through the warp's staging rows, then contiguous row stores
            const int col = c0 + lane;
            const int pos = col;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
            {
#pragma unroll
                for (int nt = 0; nt < NTG; ++nt)
                    *reinterpret_cast<double2 *>(stg + g * LDS_STAGE + nt * 8 + 2 * t) = make_double2(acc[mt][nt][0], acc[mt][nt][1]);
                __syncwarp();
                if (lane < GW && col < n_cols)
                {
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                    {
                        const int el = mt * 8 + r;
                        if (el < n_e)
                        {
                            double *row = a.M + (e0 + el) * nc;
                            const double v = stg[r * LDS_STAGE + lane];
                            double v1 = v;
                            if (a.op == ACRO_B200_OP_ADD) v1 = row[pos] + v;
                            else if (a.op == ACRO_B200_OP_SUB) v1 = row[pos] - v;
                            __stcs(row + pos, v1);
                        }
                    }
                }
                __syncwarp();
            }
        }
        __syncthreads();   // every warp is done with this W buffer
        buf ^= 1;
    }
}


// ------------------------------------------------------------------ symmetric variant
// B1 == B2: only the packed columns (i <= j) are computed.  The warps of a CTA share one
// tile of MT*8 elements; warp w owns column tiles NTW*w .. NTW*w+NTW-1 for all MT row tiles.
// Results are scattered, entry (i,j) and its mirror (j,i), into a shared-memory image of 8
// full element matrices, which then leaves as ONE contiguous bulk store; IMAGES such images
// alternate so the store of one row tile drains while the next is scattered.
// Measured on B200 (E = 2^18, 27 x 27): 8 warps x 6 column tiles x 2 row tiles, 1 image, two
// CTAs per SM (one CTA's scatter/store overlaps the other's tensor-core loop): 0.566 ms;
// 16 warps x 3 x 4, 2 images, one CTA per SM: 0.579 ms; 8 warps x 6 x 4, 2 images, one CTA:
// 0.601 ms.  Recomputing the mirror positions in the epilogue (integer divisions) instead of
// keeping them in registers costs 0.08 ms.  Shared-memory wavefronts (fragment loads, scatter,
// bulk store) are about as many as tensor-pipe cycles, which is what bounds all three.
template <int WARPS_, int NTW_, int MT_, int IMAGES_, int CTAS_>
struct SymCfg
{
    static constexpr int WARPS = WARPS_, NTW = NTW_, MT = MT_, IMAGES = IMAGES_, CTAS = CTAS_;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int TILE_E = MT * 8;                 // elements per tile
    static constexpr int MAX_COLS = WARPS * NTW * 8;      // packed columns covered
};

struct SymLayout
{
    int ldb, b_off, stage_off, stage_bytes, bar_off, total;     // byte offsets into dynamic shared memory
};

__host__ __device__ inline SymLayout sym_layout(int ni, int tile_e, int images)
{
    SymLayout l;
    l.ldb = ni;
    while (l.ldb % 8 != 4) ++l.ldb;                        // row stride = 4 mod 8 doubles: fewer bank conflicts in fragment loads
    const int w_bytes = 2 * tile_e * LDW * 8;
    l.b_off = w_bytes;
    const int b_bytes = ((QN * l.ldb * 8 + 127) / 128) * 128;
    l.stage_off = l.b_off + b_bytes;
    l.stage_bytes = ((8 * ni * ni * 8 + 127) / 128) * 128;
    l.bar_off = l.stage_off + images * l.stage_bytes;
    l.total = l.bar_off + 64;
    return l;
}

// QC: the contracted extent when known at compile time (64), 0 = taken from the arguments.
template <class C, int QC>
__global__ void __launch_bounds__(C::THREADS, C::CTAS)
rank1_gemm_sym_kernel(const Rank1Args a)
{
    const int q_ext = QC > 0 ? QC : (a.q + 3) & ~3;     // steps of four; the padding rows / columns are zero
    constexpr int NTW = C::NTW, MT = C::MT, TE = C::TILE_E, THREADS = C::THREADS;
    extern __shared__ __align__(128) unsigned char raw[];
    const int ni = a.ni, nc = ni * ni, n_cols = ni * (ni + 1) / 2;
    const SymLayout L = sym_layout(ni, TE, C::IMAGES);
    const int ldb = L.ldb;
    double *sW = reinterpret_cast<double *>(raw);                        // [2][TE * LDW]
    double *sB = reinterpret_cast<double *>(raw + L.b_off);             // [QN][ldb]
    uint64_t *full = reinterpret_cast<uint64_t *>(raw + L.bar_off);     // [2]

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n_tiles = (a.elements + TE - 1) / TE;

    if (tid == 0)
    {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        fence_mbar_init();
    }
    for (int i = tid; i < q_ext * ni; i += THREADS) sB[(i / ni) * ldb + (i % ni)] = i < a.q * ni ? a.B1[i] : 0.0;
    for (int i = tid; i < 2 * TE * (q_ext - a.q); i += THREADS)
        sW[(i / (q_ext - a.q)) * LDW + a.q + i % (q_ext - a.q)] = 0.0;
    __syncthreads();

    // packed column c -> (i, j), row-major upper triangle; fixed per thread for the whole kernel
    auto unpack = [&](int c, int &i, int &j) {
        int row = 0, start = 0;
        while (start + (ni - row) <= c) { start += ni - row; ++row; }
        i = row;
        j = row + (c - start);
    };
    int off1[NTW], off2[NTW];    // B-fragment column of this lane
    int pos_d[NTW][2], pos_m[NTW][2];   // where this lane's two C-fragment columns and their mirrors go (-1: padding)
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt)
    {
        const int cbase = (warp * NTW + nt) * 8;
        int c = cbase + g;
        c = c < n_cols ? c : n_cols - 1;        // padded columns compute a copy that is never stored
        unpack(c, off1[nt], off2[nt]);
#pragma unroll
        for (int h = 0; h < 2; ++h)
        {
            const int cc = cbase + 2 * t + h;
            pos_d[nt][h] = pos_m[nt][h] = -1;
            if (cc < n_cols)
            {
                int i, j;
                unpack(cc, i, j);
                pos_d[nt][h] = i * ni + j;
                if (i != j) pos_m[nt][h] = j * ni + i;
            }
        }
    }

    auto issue_w = [&](int64_t tile, int buf) {
        const int64_t e0 = tile * TE;
        if (!a.use_bulk || e0 >= a.elements) return;
        if (tid < 32)
        {
            const int64_t left = a.elements - e0;
            const int n_e = left < TE ? static_cast<int>(left) : TE;
            if (tid == 0) mbar_arrive_expect_tx(&full[buf], n_e * a.q * 8);
            __syncwarp();
            if (tid < n_e) bulk_load(sW + buf * TE * LDW + tid * LDW, a.W + (e0 + tid) * a.q, a.q * 8, &full[buf]);
        }
    };

    int64_t tile = blockIdx.x;
    issue_w(tile, 0);
    uint32_t phase_bits = 0;
    int buf = 0;
    uint32_t images = 0;   // row-tile images written so far (selects the staging buffer)
    const bool bulk_out = aligned16(a.M);

    for (; tile < n_tiles; tile += gridDim.x)
    {
        issue_w(tile + gridDim.x, buf ^ 1);
        const int64_t e0 = tile * TE;
        const int64_t left = a.elements - e0;
        const int n_e = left < TE ? static_cast<int>(left) : TE;
        if (a.use_bulk)
        {
            if (!mbar_wait(&full[buf], (phase_bits >> buf) & 1u)) atomicExch(a.wait_flag, 1);
            phase_bits ^= (1u << buf);
        }
        else
        {
            for (int i = tid; i < n_e * a.q; i += THREADS) sW[buf * TE * LDW + (i / a.q) * LDW + (i % a.q)] = __ldcs(a.W + e0 * a.q + i);
            __syncthreads();
        }
        const double *sw = sW + buf * TE * LDW;

        double acc[MT][NTW][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = 0.0;
#pragma unroll 2
        for (int k0 = 0; k0 < q_ext; k0 += 4)
        {
            double af[MT], bf[NTW];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) af[mt] = sw[(mt * 8 + g) * LDW + k0 + t];
            const double *b = sB + (k0 + t) * ldb;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) bf[nt] = b[off1[nt]] * b[off2[nt]];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTW; ++nt) dmma_m8n8k4(acc[mt][nt], af[mt], bf[nt]);
        }

#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
            const int rows = n_e - mt * 8 < 8 ? (n_e - mt * 8 > 0 ? n_e - mt * 8 : 0) : 8;   // valid elements of this row tile
            double *img = reinterpret_cast<double *>(raw + L.stage_off + (images % C::IMAGES) * L.stage_bytes);
            // the image buffer was last stored IMAGES images ago: all newer stores may still be draining
            if (tid == 0 && images >= C::IMAGES) bulk_wait_read<C::IMAGES - 1>();
            __syncthreads();
            double *row = img + g * nc;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    if (pos_d[nt][h] >= 0) row[pos_d[nt][h]] = acc[mt][nt][h];
                    if (pos_m[nt][h] >= 0) row[pos_m[nt][h]] = acc[mt][nt][h];
                }
            fence_proxy_async();
            __syncthreads();
            double *dst = a.M + (e0 + mt * 8) * nc;
            if (bulk_out && rows == 8)
            {
                if (tid == 0)
                {
                    bulk_store(dst, img, 8 * nc * 8);
                    bulk_commit();
                }
            }
            else
            {
                for (int i = tid; i < rows * nc; i += THREADS) __stcs(dst + i, img[i]);
                if (tid == 0) bulk_commit();   // an empty group keeps the image/store numbering in step
            }
            ++images;
        }
        buf ^= 1;
    }
    if (tid == 0) bulk_wait_all<0>();   // shared memory must outlive the stores that read it
}

// ------------------------------------------------------------------ symmetric variant, right operand in tensor memory
// The same packed-column scheme, with the formed right operand BB[q,(i,j)] = B[q,i]*B[q,j] kept on chip for
// the whole launch instead of being formed again for every tile.  For 27 x 27 and 64 quadrature points it is
// 64 x 384 doubles = 192 KB: more than the register file or shared memory can spare, but it fits the SM's
// 256 KB of tensor memory, which registers reach through a path of their own (tmem.cuh).  Every thread parks
// the 96 fragment entries it needs (16 k-steps x 6 column tiles) once and reads them back, twelve per pair of
// k-steps, in front of the tensor-core instructions that consume them.  That removes the two shared-memory
// loads and the multiply per fragment entry from the inner loop, whose shared-memory traffic was as large as
// its tensor-pipe time (the old variant measured 58 % tensor-pipe activity with the shared-memory pipe at
// 57 % and conflicts on top): what is left there is the W fragment.
//
// One CTA of 16 warps per SM, as two groups of 8 warps.  A group works like a CTA of the old variant (its own
// stream of 16-element tiles, W double buffer, image and bulk store, synchronised by a named barrier), so one
// group's scatter and store overlap the other's tensor-core loop; warp w of either group uses the same
// columns, so both groups read the one copy of BB (each group writes half of its k-steps).
constexpr int TM_GROUPS = 2, TM_GROUP_WARPS = 8, TM_GROUP_THREADS = TM_GROUP_WARPS * 32, TM_THREADS = TM_GROUPS * TM_GROUP_THREADS;
constexpr int TM_NTW = 6, TM_MT = 2, TM_TE = TM_MT * 8;
constexpr int TM_MAX_COLS = TM_GROUP_WARPS * TM_NTW * 8;          // 384 packed columns
static_assert(TM_NTW == 6, "the inner loop fetches six fragment entries per k-step as four plus two doubles");
constexpr int TM_WARP_COLUMNS = (QN / 4) * TM_NTW * 2;            // 192 32-bit columns per thread
constexpr uint32_t TM_ALLOC_COLUMNS = 512;
constexpr int TM_IMAGES = 2;                                        // images per group, used alternately

struct TmemSymLayout
{
    int ldb, b_off, img_off, img_bytes, bar_off, slot_off, total;     // byte offsets into dynamic shared memory
};

__host__ __device__ inline TmemSymLayout tmem_sym_layout(int ni)
{
    TmemSymLayout l;
    l.ldb = ni;
    while (l.ldb % 8 != 4) ++l.ldb;
    const int w_bytes = TM_GROUPS * 2 * TM_TE * LDW * 8;
    l.b_off = w_bytes;
    const int b_bytes = ((QN * l.ldb * 8 + 127) / 128) * 128;
    // B is needed only until the right operand is parked in tensor memory: the images take its place afterwards
    l.img_off = l.b_off;
    l.img_bytes = ((8 * ni * ni * 8 + 127) / 128) * 128;
    const int img_all = TM_GROUPS * TM_IMAGES * l.img_bytes;
    l.bar_off = l.b_off + (img_all > b_bytes ? img_all : b_bytes);
    l.slot_off = l.bar_off + TM_GROUPS * 2 * 8;
    l.total = l.slot_off + 16;
    return l;
}

template <int QC>
__global__ void __launch_bounds__(TM_THREADS, 1)
rank1_gemm_sym_tmem_kernel(const Rank1Args a)
{
    constexpr int NTW = TM_NTW, MT = TM_MT, TE = TM_TE;
    const int q_ext = QC > 0 ? QC : (a.q + 7) & ~7;     // k-steps are taken in pairs; the padding rows / columns are zero
    extern __shared__ __align__(128) unsigned char raw[];
    const int ni = a.ni, nc = ni * ni, n_cols = ni * (ni + 1) / 2;
    const TmemSymLayout L = tmem_sym_layout(ni);
    const int ldb = L.ldb;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp >> 3, wg = warp & 7, gtid = tid & (TM_GROUP_THREADS - 1);

    double *sW_all = reinterpret_cast<double *>(raw);                                   // [groups][2][TE * LDW]
    double *sW = sW_all + group * 2 * TE * LDW;
    double *sB = reinterpret_cast<double *>(raw + L.b_off);                             // [q_ext][ldb]
    unsigned char *img_base = raw + L.img_off + group * TM_IMAGES * L.img_bytes;        // [images] 8 element matrices each
    uint64_t *full = reinterpret_cast<uint64_t *>(raw + L.bar_off) + group * 2;         // [2]
    uint32_t *slot = reinterpret_cast<uint32_t *>(raw + L.slot_off);

    if (tid == 0)
    {
        for (int i = 0; i < TM_GROUPS * 2; ++i) mbar_init(reinterpret_cast<uint64_t *>(raw + L.bar_off) + i, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(slot, TM_ALLOC_COLUMNS);
    for (int i = tid; i < q_ext * ni; i += TM_THREADS) sB[(i / ni) * ldb + (i % ni)] = i < a.q * ni ? a.B1[i] : 0.0;
    {
        const int pad = q_ext - a.q;      // the W rows of all four buffers are contiguous: rows 0 .. 4*TE-1
        for (int i = tid; i < TM_GROUPS * 2 * TE * pad; i += TM_THREADS) sW_all[(i / pad) * LDW + a.q + i % pad] = 0.0;
    }
    tmem_fence_before_sync();
    __syncthreads();
    tmem_fence_after_sync();
    const uint32_t tmem_base = *slot;
    // this warp's lanes (its quarter of the 128) and its 192 columns (two warps of a group share a quarter)
    const uint32_t tcol = tmem_base + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + static_cast<uint32_t>(((warp >> 2) & 1) * TM_WARP_COLUMNS);

    // packed column c -> (i, j), row-major upper triangle; fixed per thread for the whole kernel
    auto unpack = [&](int c, int &i, int &j) {
        int row = 0, start = 0;
        while (start + (ni - row) <= c) { start += ni - row; ++row; }
        i = row;
        j = row + (c - start);
    };
    // where this lane's two C-fragment columns of every column tile and their mirrors go in an element matrix:
    // low half = position of (i,j), high half = position of (j,i); 0xFFFF = nothing to store
    uint32_t pos[NTW][2];
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt)
    {
        const int cbase = (wg * NTW + nt) * 8;
#pragma unroll
        for (int h = 0; h < 2; ++h)
        {
            const int cc = cbase + 2 * t + h;
            uint32_t direct = 0xFFFFu, mirror = 0xFFFFu;
            if (cc < n_cols)
            {
                int i, j;
                unpack(cc, i, j);
                direct = static_cast<uint32_t>(i * ni + j);
                if (i != j) mirror = static_cast<uint32_t>(j * ni + i);
            }
            pos[nt][h] = direct | (mirror << 16);
        }
    }

    {
        // park this thread's fragment entries of BB: k-step ks, column tile nt at columns 12*ks + 2*nt (+1).  Warp w of
        // either group owns the same columns, so the two groups share the work: even k-steps by group 0, odd by group 1.
        int off1[NTW], off2[NTW];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
        {
            int c = (wg * NTW + nt) * 8 + g;
            c = c < n_cols ? c : n_cols - 1;        // padded columns compute a copy that is never stored
            unpack(c, off1[nt], off2[nt]);
        }
        for (int ks = group; ks < q_ext / 4; ks += TM_GROUPS)
        {
            const double *b = sB + (4 * ks + t) * ldb;
            double v[NTW];
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) v[nt] = b[off1[nt]] * b[off2[nt]];
#pragma unroll
            for (int nt = 0; nt < NTW; nt += 2) tmem_store_2(tcol + ks * (2 * NTW) + 2 * nt, v[nt], v[nt + 1]);
        }
        tmem_wait_stores();
    }
    tmem_fence_before_sync();
    __syncthreads();
    tmem_fence_after_sync();

    const int64_t n_tiles = (a.elements + TE - 1) / TE;
    const int64_t stride = static_cast<int64_t>(TM_GROUPS) * gridDim.x;
    auto issue_w = [&](int64_t tile, int buf) {
        const int64_t e0 = tile * TE;
        if (!a.use_bulk || e0 >= a.elements) return;
        if (gtid < 32)
        {
            const int64_t left = a.elements - e0;
            const int n_e = left < TE ? static_cast<int>(left) : TE;
            if (gtid == 0) mbar_arrive_expect_tx(&full[buf], n_e * a.q * 8);
            __syncwarp();
            if (gtid < n_e) bulk_load(sW + buf * TE * LDW + gtid * LDW, a.W + (e0 + gtid) * a.q, a.q * 8, &full[buf]);
        }
    };

    int64_t tile = static_cast<int64_t>(TM_GROUPS) * blockIdx.x + group;
    issue_w(tile, 0);
    uint32_t phase_bits = 0;
    int buf = 0;
    uint32_t round = 0;       // row tiles this group has finished (selects the image)
    // The two groups should run half a tile apart, one in its tensor-core loop while the other scatters and stores.
    // Left alone they start together and only drift apart over many tiles; short launches never get there.  So group 1
    // holds its first tile back until group 0 is half-way through the k-steps of its own first tile (named barrier 3,
    // group 0 arriving without blocking; it arrives after its loop at the latest, so group 1 cannot be left waiting).
    bool stagger_pending = true;
    const bool bulk_out = aligned16(a.M);
    const int bar_id = 1 + group;

    for (; tile < n_tiles; tile += stride)
    {
        issue_w(tile + stride, buf ^ 1);     // released by the barriers that closed the previous tile
        const int64_t e0 = tile * TE;
        const int64_t left = a.elements - e0;
        const int n_e = left < TE ? static_cast<int>(left) : TE;
        if (a.use_bulk)
        {
            if (!mbar_wait(&full[buf], (phase_bits >> buf) & 1u)) atomicExch(a.wait_flag, 1);
            phase_bits ^= (1u << buf);
        }
        else
        {
            for (int i = gtid; i < n_e * a.q; i += TM_GROUP_THREADS) sW[buf * TE * LDW + (i / a.q) * LDW + (i % a.q)] = __ldcs(a.W + e0 * a.q + i);
            named_barrier(bar_id, TM_GROUP_THREADS);
        }
        const double *sw = sW + buf * TE * LDW;
        if (group == 1 && stagger_pending)
        {
            named_barrier(3, TM_THREADS);
            stagger_pending = false;
        }

        double acc[MT][NTW][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = 0.0;
        // Twelve fragment entries (two k-steps x six column tiles) per fetch from tensor memory; the fetch latency is
        // covered by the other warps of the SM sub-partition (fetching one k-step ahead into a second register set
        // was measured 3 % slower).
#pragma unroll 2
        for (int kp = 0; kp < q_ext / 8; ++kp)
        {
            if (group == 0 && stagger_pending && kp == q_ext / 16)
            {
                named_barrier_arrive(3, TM_THREADS);
                stagger_pending = false;
            }
            uint32_t fa[8], fb[8], fc[8];      // doubles 0..3, 4..7, 8..11: k-step 2*kp (0..5), then k-step 2*kp+1 (6..11)
            tmem_load_4(tcol + kp * (4 * NTW), fa);
            tmem_load_4(tcol + kp * (4 * NTW) + 8, fb);
            tmem_load_4(tcol + kp * (4 * NTW) + 16, fc);
            double af[2][MT];
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) af[s2][mt] = sw[(mt * 8 + g) * LDW + kp * 8 + s2 * 4 + t];
            tmem_wait_loads();
            double bf[2][NTW];
#pragma unroll
            for (int d = 0; d < 4; ++d)
            {
                bf[0][d] = tmem_double(fa[2 * d], fa[2 * d + 1]);
                (d < 2 ? bf[0][4 + d] : bf[1][d - 2]) = tmem_double(fb[2 * d], fb[2 * d + 1]);
                bf[1][2 + d] = tmem_double(fc[2 * d], fc[2 * d + 1]);
            }
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NTW; ++nt) dmma_m8n8k4(acc[mt][nt], af[s2][mt], bf[s2][nt]);
        }

#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
        {
            const int rows = n_e - mt * 8 < 8 ? (n_e - mt * 8 > 0 ? n_e - mt * 8 : 0) : 8;   // valid elements of this row tile
            // Row tile r goes through image r % 2.  The last store that read this image belongs to row tile r - 2; thread 0
            // waited for it before the barrier of row tile r - 1, so every thread may write here without another barrier.
            double *img = reinterpret_cast<double *>(img_base + (round % TM_IMAGES) * L.img_bytes);
            double *row = img + g * nc;
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    const uint32_t direct = pos[nt][h] & 0xFFFFu, mirror = pos[nt][h] >> 16;
                    if (direct != 0xFFFFu) row[direct] = acc[mt][nt][h];
                    if (mirror != 0xFFFFu) row[mirror] = acc[mt][nt][h];
                }
            fence_proxy_async();
            if (gtid == 0) bulk_wait_read<0>();      // the store of the previous row tile (the other image) has read its image
            named_barrier(bar_id, TM_GROUP_THREADS);
            double *dst = a.M + (e0 + mt * 8) * nc;
            if (bulk_out && rows == 8)
            {
                if (gtid == 0)
                {
                    bulk_store(dst, img, 8 * nc * 8);
                    bulk_commit();
                }
            }
            else
            {
                for (int i = gtid; i < rows * nc; i += TM_GROUP_THREADS) __stcs(dst + i, img[i]);
                named_barrier(bar_id, TM_GROUP_THREADS);     // plain loads of the image: finished before it is written again
            }
            ++round;
        }
        buf ^= 1;
    }
    if (group == 0 && stagger_pending) named_barrier_arrive(3, TM_THREADS);     // no tile for this group at all
    if (gtid == 0) bulk_wait_all<0>();   // shared memory must outlive the stores that read it
    tmem_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_free(tmem_base, TM_ALLOC_COLUMNS);
}

typedef SymCfg<8, 6, 2, 1, 2> SymSmall;    // 256 threads, 16-element tiles, one image, two CTAs per SM

}

extern "C" {

int acro_b200_rank1_gemm_supported(int q, int ni, int nj)
{
    return (q >= 1 && q <= QN && ni >= 1 && ni <= MAXN && nj >= 1 && nj <= MAXN) ? 1 : 0;
}

int acro_b200_rank1_gemm(const double *W, const double *B1, const double *B2, double *M, int64_t elements, int q, int ni, int nj,
                         int op, void *stream)
{
    if (W == nullptr || B1 == nullptr || B2 == nullptr || M == nullptr) return fail_invalid("acro_b200_rank1_gemm: null argument");
    if (elements < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_rank1_gemm: bad element count or operator");
    if (!acro_b200_rank1_gemm_supported(q, ni, nj)) return fail_unsupported("acro_b200_rank1_gemm: needs 1 <= q <= 64 and 1 <= ni, nj <= 32");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_rank1_gemm");

    Rank1Args args;
    args.W = W;
    args.B1 = B1;
    args.B2 = B2;
    args.M = M;
    args.elements = elements;
    args.q = q;
    args.ni = ni;
    args.nj = nj;
    args.op = op;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_rank1_gemm (status flag)");
    args.use_bulk = (aligned16(W) && q % 2 == 0) ? 1 : 0;     // a W row must be a 16-byte multiple to travel as a bulk copy

    const size_t smem = sizeof(Smem);
    const int64_t n_tiles = (elements + ET - 1) / ET;
    static_assert(TM_MAX_COLS == SymSmall::MAX_COLS, "both symmetric variants cover the same packed columns");
    const bool symmetric = (B1 == B2 && ni == nj && op == ACRO_B200_OP_ASSIGN && ni * (ni + 1) / 2 <= TM_MAX_COLS);
    static const bool old_variant = [] { const char *e = std::getenv("ACRO_B200_RANK1_OLD"); return e != nullptr && e[0] == '1'; }();
    if (symmetric && !old_variant)
    {
        const TmemSymLayout L = tmem_sym_layout(ni);
        auto tm_kernel = q == QN ? rank1_gemm_sym_tmem_kernel<QN> : rank1_gemm_sym_tmem_kernel<0>;
        cudaError_t st = cudaFuncSetAttribute(tm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
        if (st != cudaSuccess) return fail_cuda(st, "acro_b200_rank1_gemm (shared memory opt-in)");
        const int64_t sym_tiles = (elements + TM_TE - 1) / TM_TE;
        int64_t g1 = sms;
        if (g1 > (sym_tiles + TM_GROUPS - 1) / TM_GROUPS) g1 = (sym_tiles + TM_GROUPS - 1) / TM_GROUPS;
        tm_kernel<<<static_cast<int>(g1), TM_THREADS, L.total, as_stream(stream)>>>(args);
        return launch_status("acro_b200_rank1_gemm (symmetric, tensor memory)");
    }
    if (symmetric)
    {
        const SymLayout L = sym_layout(ni, SymSmall::TILE_E, SymSmall::IMAGES);
        auto sym_kernel = q == QN ? rank1_gemm_sym_kernel<SymSmall, QN> : rank1_gemm_sym_kernel<SymSmall, 0>;
        cudaError_t st = cudaFuncSetAttribute(sym_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
        if (st != cudaSuccess) return fail_cuda(st, "acro_b200_rank1_gemm (shared memory opt-in)");
        const int64_t sym_tiles = (elements + SymSmall::TILE_E - 1) / SymSmall::TILE_E;
        int64_t g1 = static_cast<int64_t>(sms) * SymSmall::CTAS;
        if (g1 > sym_tiles) g1 = sym_tiles;
        sym_kernel<<<static_cast<int>(g1), SymSmall::THREADS, L.total, as_stream(stream)>>>(args);
        return launch_status("acro_b200_rank1_gemm (symmetric)");
    }
    auto kernel = rank1_gemm_kernel<4>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_rank1_gemm (shared memory opt-in)");
    int64_t grid = static_cast<int64_t>(sms) * 2;
    if (grid > n_tiles) grid = n_tiles;
    kernel<<<static_cast<int>(grid), NTHREADS, smem, as_stream(stream)>>>(args);
    return launch_status("acro_b200_rank1_gemm");
}

}
