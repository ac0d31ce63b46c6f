// sumfact_mass: the six-stage sum-factorised 3D mass operator, fused into one kernel.
//
//   T1_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3        Y1_e_i1_k2_k3 = B_k1_i1 X_e_k1_k2_k3
//   T2_e_i1_k2_k3 = B_k2_i2 T1_e_i1_i2_k3       Y2_e_i1_i2_k3 = B_k2_i2 Y1_e_i1_k2_k3
//   X_e_k1_k2_k3  = B_k1_i1 T2_e_i1_k2_k3 W_e_k1_k2_k3      V_e_i1_i2_i3 = B_k3_i3 Y2_e_i1_i2_k3
//
// Only U, W (read) and V (written) touch HBM: 8*(P^3 + Q^3 + P^3) = 2024 bytes per element
// for P = 4 dofs, Q = 5 quadrature points per direction; T1, T2, X, Y1 live in registers and
// Y2 crosses threads once through shared memory.
//
// Work split: Q threads per element.  Thread (e, k3) owns the k3-plane: stages 1-5 contract
// i3, i2, i1, k1, k2 entirely in its registers (U is read from shared memory, the Q threads
// of an element reading the same address in the same instruction: a broadcast).  Stage 6
// contracts k3, which crosses the plane owners: Y2 goes through shared memory and thread
// (e, i1) finishes V_e_i1_*_* and writes it over its own Y2 slots (read into registers
// first), so V needs no buffer of its own and three CTAs fit on an SM.  Tiles of 32 elements; U and W tiles arrive by asynchronous
// bulk copies (per element for U, into slots padded by two doubles so that the elements of a
// warp fall into different banks, or one span when the element size is odd; one span for W), issued as soon as the previous tile's
// copies are dead, so they overlap the rest of that tile and the other CTA of the SM.
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int ET = 32;   // elements per tile

// Compile-time geometry for P dofs and Q quadrature points per direction.
template <int P_, int Q_, int CTAS_>
struct Geo
{
    static constexpr int P = P_, Q = Q_, CTAS = CTAS_;
    static constexpr int NT = ET * Q;                                 // threads per CTA
    static constexpr int U_ELEM = P * P * P, W_ELEM = Q * Q * Q;
    // Even element size: slots padded by two doubles, so that the elements of a warp fall into different
    // banks and every slot stays a 16-byte multiple (one bulk copy per element).  Odd element size: the
    // unpadded odd stride is already conflict-free, and the tile travels as one contiguous span.
    static constexpr bool U_ODD = (U_ELEM % 2 != 0);
    static constexpr int U_STRIDE = U_ODD ? U_ELEM : U_ELEM + 2;
    static constexpr int Y_ROW = P * Q;                               // Y2 row of one (element, i1); V reuses the first P*P
    static constexpr int Y_MIN = P * P * Q;
    static constexpr int Y_STRIDE = Y_MIN + ((Q - Y_MIN % 16) % 16 + 16) % 16;   // = Q mod 16: plane owners of a half warp hit distinct banks
};

template <class G>
struct Smem
{
    double U[ET * G::U_STRIDE];
    double W[ET * G::W_ELEM];
    double Y[ET * G::Y_STRIDE];
    double B[G::Q * G::P];
    uint64_t bar;
};

struct MassArgs
{
    const double *B;
    const double *U;
    const double *W;
    double *V;
    int64_t elements;
    int *wait_flag;
    int use_bulk;   // operands are 16-byte aligned: bulk copies allowed
};

template <class G>
__device__ __forceinline__ void issue_tile_load(Smem<G> &s, const MassArgs &a, int64_t tile, int64_t n_tiles_full)
{
    // Only whole tiles travel by bulk copy (sizes and addresses stay 16-byte multiples).
    if (!a.use_bulk || tile >= n_tiles_full) return;
    if (threadIdx.x < 32)
    {
        const int64_t e0 = tile * ET;
        if (threadIdx.x == 0) mbar_arrive_expect_tx(&s.bar, ET * (G::U_ELEM + G::W_ELEM) * 8);
        __syncwarp();
        if (!G::U_ODD) bulk_load(s.U + threadIdx.x * G::U_STRIDE, a.U + (e0 + threadIdx.x) * G::U_ELEM, G::U_ELEM * 8, &s.bar);
        else if (threadIdx.x == 0) bulk_load(s.U, a.U + e0 * G::U_ELEM, ET * G::U_ELEM * 8, &s.bar);
        if (threadIdx.x == 0) bulk_load(s.W, a.W + e0 * G::W_ELEM, ET * G::W_ELEM * 8, &s.bar);
    }
}

template <class G>
__global__ void __launch_bounds__(G::NT, G::CTAS)
sumfact_mass_kernel(const MassArgs a)
{
    constexpr int P = G::P, Q = G::Q, NT = G::NT;
    constexpr int U_ELEM = G::U_ELEM, W_ELEM = G::W_ELEM, U_STRIDE = G::U_STRIDE, Y_STRIDE = G::Y_STRIDE, Y_ROW = G::Y_ROW;
    extern __shared__ __align__(128) unsigned char raw[];
    Smem<G> &s = *reinterpret_cast<Smem<G> *>(raw);
    const int tid = threadIdx.x;
    const int64_t n_tiles = (a.elements + ET - 1) / ET;
    const int64_t n_tiles_full = a.elements / ET;

    if (tid == 0)
    {
        mbar_init(&s.bar, 1);
        fence_mbar_init();
    }
    if (tid < Q * P) s.B[tid] = a.B[tid];
    __syncthreads();

    double Bm[Q][P];   // B_k_i
#pragma unroll
    for (int k = 0; k < Q; ++k)
#pragma unroll
        for (int i = 0; i < P; ++i) Bm[k][i] = s.B[k * P + i];

    // plane ownership (stages 1-5) and row ownership (stage 6)
    const int eb = tid / Q, k3 = tid % Q;
    const int ec = tid / P, i1c = tid % P;
    double brow[P];   // B_k3_*
#pragma unroll
    for (int i = 0; i < P; ++i) brow[i] = s.B[k3 * P + i];

    uint32_t parity = 0;
    int64_t tile = blockIdx.x;
    issue_tile_load(s, a, tile, n_tiles_full);

    for (; tile < n_tiles; tile += gridDim.x)
    {
        const int64_t e0 = tile * ET;
        const int64_t left = a.elements - e0;
        const int n_e = left < ET ? static_cast<int>(left) : ET;
        const bool by_bulk = a.use_bulk && tile < n_tiles_full;

        if (!by_bulk)
        {
            // plain coalesced loads (ragged or unaligned tile)
            for (int i = tid; i < n_e * U_ELEM; i += NT) s.U[(i / U_ELEM) * U_STRIDE + (i % U_ELEM)] = __ldcs(a.U + e0 * U_ELEM + i);
            for (int i = tid; i < n_e * W_ELEM; i += NT) s.W[i] = __ldcs(a.W + e0 * W_ELEM + i);
            __syncthreads();
        }
        else
        {
            if (!mbar_wait(&s.bar, parity)) atomicExch(a.wait_flag, 1);
            parity ^= 1u;
        }

        if (eb < n_e)
        {
            const double *u = s.U + eb * U_STRIDE;
            // stage 1: T1_i1_i2 (this k3) = sum_i3 B_k3_i3 U_i1_i2_i3
            double t1[P][P];
#pragma unroll
            for (int i1 = 0; i1 < P; ++i1)
#pragma unroll
                for (int i2 = 0; i2 < P; ++i2)
                {
                    const double *ur = u + (i1 * P + i2) * P;
                    double uv[P];
                    if (P % 2 == 0)
                    {
                        // even P: rows of U start on 16-byte boundaries in the padded slot
#pragma unroll
                        for (int i3 = 0; i3 < P; i3 += 2)
                        {
                            const double2 pair = *reinterpret_cast<const double2 *>(ur + i3);
                            uv[i3] = pair.x;
                            uv[i3 + 1 < P ? i3 + 1 : i3] = pair.y;
                        }
                    }
                    else
                    {
#pragma unroll
                        for (int i3 = 0; i3 < P; ++i3) uv[i3] = ur[i3];
                    }
                    double acc = brow[0] * uv[0];
#pragma unroll
                    for (int i3 = 1; i3 < P; ++i3) acc = fma(brow[i3], uv[i3], acc);
                    t1[i1][i2] = acc;
                }
            // stage 2: T2_i1_k2 = sum_i2 B_k2_i2 T1_i1_i2
            double t2[P][Q];
#pragma unroll
            for (int i1 = 0; i1 < P; ++i1)
#pragma unroll
                for (int k2 = 0; k2 < Q; ++k2)
                {
                    double acc = Bm[k2][0] * t1[i1][0];
#pragma unroll
                    for (int i2 = 1; i2 < P; ++i2) acc = fma(Bm[k2][i2], t1[i1][i2], acc);
                    t2[i1][k2] = acc;
                }
            // stage 3: X_k1_k2 = W_k1_k2_k3 * sum_i1 B_k1_i1 T2_i1_k2
            double x[Q][Q];
            const double *w = s.W + eb * W_ELEM + k3;
#pragma unroll
            for (int k1 = 0; k1 < Q; ++k1)
#pragma unroll
                for (int k2 = 0; k2 < Q; ++k2)
                {
                    double acc = Bm[k1][0] * t2[0][k2];
#pragma unroll
                    for (int i1 = 1; i1 < P; ++i1) acc = fma(Bm[k1][i1], t2[i1][k2], acc);
                    x[k1][k2] = acc * w[(k1 * Q + k2) * Q];
                }
            // stage 4: Y1_i1_k2 = sum_k1 B_k1_i1 X_k1_k2
            double y1[P][Q];
#pragma unroll
            for (int i1 = 0; i1 < P; ++i1)
#pragma unroll
                for (int k2 = 0; k2 < Q; ++k2)
                {
                    double acc = Bm[0][i1] * x[0][k2];
#pragma unroll
                    for (int k1 = 1; k1 < Q; ++k1) acc = fma(Bm[k1][i1], x[k1][k2], acc);
                    y1[i1][k2] = acc;
                }
            // stage 5: Y2_i1_i2 = sum_k2 B_k2_i2 Y1_i1_k2  -> shared, layout [e][i1][i2][k3]
            double *y = s.Y + eb * Y_STRIDE + k3;
#pragma unroll
            for (int i1 = 0; i1 < P; ++i1)
#pragma unroll
                for (int i2 = 0; i2 < P; ++i2)
                {
                    double acc = Bm[0][i2] * y1[i1][0];
#pragma unroll
                    for (int k2 = 1; k2 < Q; ++k2) acc = fma(Bm[k2][i2], y1[i1][k2], acc);
                    y[(i1 * P + i2) * Q] = acc;
                }
        }
        __syncthreads();   // U and W of this tile are dead, Y2 is complete
        issue_tile_load(s, a, tile + gridDim.x, n_tiles_full);

        if (ec < n_e && tid < ET * P)
        {
            // stage 6: V_i1_i2_i3 = sum_k3 B_k3_i3 Y2_i1_i2_k3, written over this thread's own Y2 row
            double *y = s.Y + ec * Y_STRIDE + i1c * Y_ROW;
            double yv[P][Q];
#pragma unroll
            for (int i2 = 0; i2 < P; ++i2)
#pragma unroll
                for (int k = 0; k < Q; ++k) yv[i2][k] = y[i2 * Q + k];
#pragma unroll
            for (int i2 = 0; i2 < P; ++i2)
#pragma unroll
                for (int i3 = 0; i3 < P; ++i3)
                {
                    double acc = Bm[0][i3] * yv[i2][0];
#pragma unroll
                    for (int k = 1; k < Q; ++k) acc = fma(Bm[k][i3], yv[i2][k], acc);
                    y[i2 * P + i3] = acc;
                }
        }
        __syncthreads();   // V tile complete (inside the Y buffer)

        // contiguous coalesced store of the V tile: entry r of element e sits at e*Y_STRIDE + (r/P^2)*Y_ROW + r%P^2
        double *dst = a.V + e0 * U_ELEM;
        for (int i = tid; i < n_e * U_ELEM; i += NT)
        {
            const int el = i / U_ELEM, r = i % U_ELEM;
            __stcs(dst + i, s.Y[el * Y_STRIDE + (r / (P * P)) * Y_ROW + (r % (P * P))]);
        }
        __syncthreads();   // the next tile's stage 5 overwrites the Y buffer
    }
}

typedef Geo<4, 5, 3> Geo45;   // p = 3 hexahedra: 4 dofs, 5 quadrature points per direction
typedef Geo<3, 4, 4> Geo34;   // p = 2
typedef Geo<2, 3, 6> Geo23;   // p = 1
typedef Geo<2, 4, 6> Geo24;   // the same orders with one more quadrature point per direction
typedef Geo<3, 5, 4> Geo35;
typedef Geo<4, 6, 2> Geo46;
typedef Geo<5, 6, 1> Geo56;   // p = 4

template <class G>
int launch_mass(const MassArgs &args, int sms, cudaStream_t stream)
{
    const size_t smem = sizeof(Smem<G>);
    // The opt-in is a per-device function attribute; setting it again is a cheap host call.
    cudaError_t status = cudaFuncSetAttribute(sumfact_mass_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_sumfact_mass (shared memory opt-in)");
    const int64_t n_tiles = (args.elements + ET - 1) / ET;
    int64_t grid = static_cast<int64_t>(sms) * G::CTAS;
    if (grid > n_tiles) grid = n_tiles;
    sumfact_mass_kernel<G><<<static_cast<int>(grid), G::NT, smem, stream>>>(args);
    return launch_status("acro_b200_sumfact_mass");
}

}

extern "C" {

int acro_b200_sumfact_mass_supported(int p, int q) { return (p >= 2 && p <= 5 && (q == p + 1 || (q == p + 2 && p <= 4))) ? 1 : 0; }

int acro_b200_sumfact_mass(const double *B, const double *U, const double *W, double *V, int64_t elements, int p, int q, void *stream)
{
    if (B == nullptr || U == nullptr || W == nullptr || V == nullptr) return fail_invalid("acro_b200_sumfact_mass: null argument");
    if (elements < 1) return fail_invalid("acro_b200_sumfact_mass: element count must be positive");
    if (!acro_b200_sumfact_mass_supported(p, q)) return fail_unsupported("acro_b200_sumfact_mass: instantiated for (p, q) = (2, 3), (2, 4), (3, 4), (3, 5), (4, 5), (4, 6), (5, 6)");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_sumfact_mass");

    MassArgs args;
    args.B = B;
    args.U = U;
    args.W = W;
    args.V = V;
    args.elements = elements;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_sumfact_mass (status flag)");
    args.use_bulk = (aligned16(U) && aligned16(W)) ? 1 : 0;
    cudaStream_t s = as_stream(stream);
    if (p == 5) return launch_mass<Geo56>(args, sms, s);
    if (p == 4) return q == 5 ? launch_mass<Geo45>(args, sms, s) : launch_mass<Geo46>(args, sms, s);
    if (p == 3) return q == 4 ? launch_mass<Geo34>(args, sms, s) : launch_mass<Geo35>(args, sms, s);
    return q == 3 ? launch_mass<Geo23>(args, sms, s) : launch_mass<Geo24>(args, sms, s);
}

}
