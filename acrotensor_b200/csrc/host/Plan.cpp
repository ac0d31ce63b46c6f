// Planner: maps a bound kernel group onto the kernel families of the C ABI.
// Matching is structural (index roles and tensor layouts), never by variable name.
#include "Plan.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>

namespace acro
{
namespace plan
{

namespace
{

typedef std::vector<std::string> Names;

Names indices_of(DimensionedKernel &k, int vari) { return vari < 0 ? k.OutputVar.IndexNames : k.InputVars[vari].IndexNames; }

bool distinct(const Names &n)
{
    Names s = n;
    std::sort(s.begin(), s.end());
    return std::adjacent_find(s.begin(), s.end()) == s.end();
}

Names concat(const Names &a, const Names &b)
{
    Names r = a;
    r.insert(r.end(), b.begin(), b.end());
    return r;
}

bool is_subsequence(const Names &small, const Names &big)
{
    std::size_t j = 0;
    for (std::size_t i = 0; i < big.size() && j < small.size(); ++i)
    {
        if (big[i] == small[j]) ++j;
    }
    return j == small.size();
}

int op_code(DimensionedKernel &k) { return k.EqOperator == "=" ? ACRO_B200_OP_ASSIGN : k.EqOperator == "+=" ? ACRO_B200_OP_ADD : ACRO_B200_OP_SUB; }

std::int64_t extent_of(DimensionedKernel &k, const std::string &idx)
{
    std::string name = idx;
    return k.GetLoopDim(name);
}

std::int64_t io_bytes(DimensionedKernel &k)
{
    std::int64_t entries = k.GetVarSize64(-1) * (k.EqOperator == "=" ? 1 : 2);
    for (int vari = 0; vari < k.GetNumInputVars(); ++vari)
    {
        bool seen = false;   // the same tensor passed twice is read once
        for (int prev = 0; prev < vari; ++prev) seen = seen || k.GetVarName(prev) == k.GetVarName(vari);
        if (!seen) entries += k.GetVarSize64(vari);
    }
    return entries * 8;
}

// ---------------------------------------------------------------- generic
Step plan_generic(DimensionedKernel &k, int ki)
{
    Step s;
    s.family = Family::Generic;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    ACROBATIC_ASSERT(k.GetNumInputVars() <= ACRO_B200_MAX_INPUTS, "Too many input tensors in kernel:  " + k.KernelStr);

    // Outer loops in the output's own dimension order (fastest last), then the
    // contracted loops in summation order.
    Names loops;
    for (const std::string &idx : k.OutputVar.IndexNames)
    {
        if (std::find(loops.begin(), loops.end(), idx) == loops.end()) loops.push_back(idx);
    }
    const int n_outer = static_cast<int>(loops.size());
    for (const std::string &idx : k.ContractionIndexNames) loops.push_back(idx);
    ACROBATIC_ASSERT(loops.size() <= ACRO_B200_MAX_LOOPS, "Too many indices in kernel:  " + k.KernelStr);

    acro_b200_generic_desc &g = s.generic;
    std::memset(&g, 0, sizeof g);
    g.n_loops = static_cast<int>(loops.size());
    g.n_outer = n_outer;
    g.n_inputs = k.GetNumInputVars();
    g.op = s.op;
    std::int64_t outer_points = 1, terms = 1;
    for (int l = 0; l < g.n_loops; ++l)
    {
        g.extent[l] = extent_of(k, loops[l]);
        (l < n_outer ? outer_points : terms) *= g.extent[l];
    }
    for (int vari = -1; vari < k.GetNumInputVars(); ++vari)
    {
        std::int64_t *step = vari < 0 ? g.out_step : g.in_step[vari];
        Names idx = indices_of(k, vari);
        for (int d = 0; d < static_cast<int>(idx.size()); ++d)
        {
            int l = static_cast<int>(std::find(loops.begin(), loops.end(), idx[d]) - loops.begin());
            step[l] += k.GetVarDimStride64(vari, d);
        }
        if (vari >= 0)
        {
            TensorRef r;
            r.ki = ki;
            r.vari = vari;
            s.ins.push_back(r);
        }
    }
    s.zero_fill_first = (s.op == ACRO_B200_OP_ASSIGN) && outer_points < k.GetVarSize64(-1);
    s.bytes = io_bytes(k);
    s.flops = outer_points * terms * k.GetNumInputVars();   // (n_in - 1) multiplies + 1 add per term
    std::ostringstream note;
    if (acro_b200_generic_uses_wide_kernel(&g)) note << "CTA per range of terms (fixed-order tree sum): " << outer_points << " entries x " << terms << " terms";
    else
    {
        int blocked_loop = -1;
        const int per_thread = acro_b200_generic_blocking(&g, &blocked_loop);
        if (per_thread > 1)
        {
            note << "thread per " << per_thread << " output entries along " << loops[blocked_loop] << ": " << outer_points
                 << " entries x " << terms << " terms";
        }
        else note << "thread per output entry: " << outer_points << " entries x " << terms << " terms";
    }
    s.note = note.str();
    return s;
}

// ---------------------------------------------------------------- reduce_batch
// out_F = sum_n A_n_F [w_n]: one contracted index n that is the leading dimension of a
// "row" operand whose remaining dimensions are exactly the output's.
bool plan_reduce_batch(DimensionedKernel &k, int ki, Step &s)
{
    if (k.ContractionIndexNames.size() != 1 || !distinct(k.OutputVar.IndexNames)) return false;
    if (k.GetNumInputVars() < 1 || k.GetNumInputVars() > 2) return false;
    const std::string n = k.ContractionIndexNames[0];
    const Names row_shape = concat(Names(1, n), k.OutputVar.IndexNames);
    int row_var = -1, weight_var = -1;
    for (int vari = 0; vari < k.GetNumInputVars(); ++vari)
    {
        Names idx = indices_of(k, vari);
        if (idx == row_shape && row_var < 0) row_var = vari;
        else if (idx == Names(1, n) && weight_var < 0) weight_var = vari;
        else return false;
    }
    if (row_var < 0) return false;
    const std::int64_t rows = extent_of(k, n);
    const std::int64_t F = k.GetVarSize64(-1);
    if (F > 1024 || !acro_b200_reduce_batch_supported(rows, static_cast<int>(F))) return false;

    s = Step();
    s.family = Family::ReduceBatch;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    s.rows = rows;
    s.sizes[0] = static_cast<int>(F);
    TensorRef a;
    a.ki = ki;
    a.vari = row_var;
    s.ins.push_back(a);
    if (weight_var >= 0)
    {
        TensorRef w;
        w.ki = ki;
        w.vari = weight_var;
        s.ins.push_back(w);
    }
    s.bytes = rows * 8 * (F + (weight_var >= 0 ? 1 : 0)) + F * 8;
    s.flops = rows * F * (weight_var >= 0 ? 2 : 1);
    std::ostringstream note;
    note << "streaming reduction over " << rows << " rows of " << F << " entries"
         << (weight_var >= 0 ? ", weighted" : "") << "; fixed-order two-level combine";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- pointwise_sym
// D_<lead>_m_n_<trail> = (factors over the points, left to right) X_<lead>_<trail>_a_l Y_<lead>_<trail>_b_l
// with {a, b} = {m, n}, the factors first in the string.  <trail> empty is the point-major
// layout (D_e_k_m_n); a non-empty <trail> is the cell-major layout of the reference's own
// partial-assembly tests (D_e_m_n_k1_k2_k3).
bool plan_pointwise_sym(DimensionedKernel &k, int ki, Step &s)
{
    const Names out = k.OutputVar.IndexNames;
    if (k.ContractionIndexNames.size() != 1 || out.size() < 3 || !distinct(out)) return false;
    const int nin = k.GetNumInputVars();
    if (nin < 2 || nin - 2 > ACRO_B200_MAX_SCALARS) return false;
    const std::string l = k.ContractionIndexNames[0];
    const Names xs = indices_of(k, nin - 2), ys = indices_of(k, nin - 1);
    if (xs.size() < 3 || xs.size() != ys.size() || xs.back() != l || ys.back() != l) return false;
    const Names P(xs.begin(), xs.end() - 2);            // the point loops, in operand order
    if (Names(ys.begin(), ys.end() - 2) != P || P.empty() || P.size() > ACRO_B200_MAX_POINT_LOOPS || !distinct(P)) return false;
    const std::string a = xs[xs.size() - 2], b = ys[ys.size() - 2];
    if (a == b || a == l || b == l) return false;
    // m, n adjacent in the output; what precedes and follows them must spell P
    std::size_t pos = 0;
    while (pos + 1 < out.size() && !((out[pos] == a && out[pos + 1] == b) || (out[pos] == b && out[pos + 1] == a))) ++pos;
    if (pos + 1 >= out.size()) return false;
    const Names lead(out.begin(), out.begin() + pos), trail(out.begin() + pos + 2, out.end());
    if (concat(lead, trail) != P) return false;
    const bool swapped = (out[pos] == b);               // the first block operand carries n
    const std::int64_t dim = extent_of(k, a);
    if (extent_of(k, b) != dim || extent_of(k, l) != dim) return false;

    s = Step();
    acro_b200_pointwise_desc &d = s.pointwise;
    std::memset(&d, 0, sizeof d);
    d.dim = static_cast<int>(dim);
    d.op = op_code(k);
    d.n_point_loops = static_cast<int>(P.size());
    d.n_scalars = nin - 2;
    d.swapped = swapped ? 1 : 0;
    d.cell_points = 1;
    for (const std::string &idx : trail) d.cell_points *= extent_of(k, idx);
    std::int64_t points = 1;
    for (std::size_t j = 0; j < P.size(); ++j)
    {
        d.point_extent[j] = extent_of(k, P[j]);
        points *= d.point_extent[j];
    }
    std::int64_t scalar_entries = 0;
    for (int vari = 0; vari < nin - 2; ++vari)
    {
        Names idx = indices_of(k, vari);
        if (!distinct(idx) || !is_subsequence(idx, P)) return false;
        for (int dd = 0; dd < static_cast<int>(idx.size()); ++dd)
        {
            int j = static_cast<int>(std::find(P.begin(), P.end(), idx[dd]) - P.begin());
            d.scalar_step[vari][j] = k.GetVarDimStride64(vari, dd);
        }
        scalar_entries += k.GetVarSize64(vari);
        TensorRef r;
        r.ki = ki;
        r.vari = vari;
        s.ins.push_back(r);
    }
    if (!acro_b200_pointwise_sym_supported(&d)) return false;
    TensorRef x, y;
    x.ki = y.ki = ki;
    x.vari = nin - 2;
    y.vari = nin - 1;
    s.ins.push_back(x);
    s.ins.push_back(y);
    s.family = Family::PointwiseSym;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = d.op;
    s.rows = points;
    const bool same_xy = k.GetVarName(nin - 2) == k.GetVarName(nin - 1);
    s.bytes = 8 * (points * dim * dim * ((same_xy ? 1 : 2) + (s.op == ACRO_B200_OP_ASSIGN ? 1 : 2)) + scalar_entries);
    s.flops = points * dim * dim * dim * (nin);   // (nin-1) multiplies + 1 add per term
    std::ostringstream note;
    note << points << " points, " << dim << "x" << dim << " block per point, " << d.n_scalars << " point-wise factors, "
         << (d.cell_points > 1 ? "cell-major output (" + std::to_string(d.cell_points) + " points per cell)" : std::string("point-major output"))
         << (swapped ? ", block transposed" : "") << "; tiles through a ring of asynchronous bulk copies";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- rank1_gemm
// M_e_i_j = W_e_q B1_q_i B2_q_j (the three inputs in any order).
bool plan_rank1_gemm(DimensionedKernel &k, int ki, Step &s)
{
    const Names out = k.OutputVar.IndexNames;
    if (out.size() != 3 || !distinct(out) || k.ContractionIndexNames.size() != 1 || k.GetNumInputVars() != 3) return false;
    const std::string e = out[0], i = out[1], j = out[2], q = k.ContractionIndexNames[0];
    int w = -1, b1 = -1, b2 = -1;
    for (int vari = 0; vari < 3; ++vari)
    {
        const Names idx = indices_of(k, vari);
        if (idx == Names{e, q} && w < 0) w = vari;
        else if (idx == Names{q, i} && b1 < 0) b1 = vari;
        else if (idx == Names{q, j} && b2 < 0) b2 = vari;
        else return false;
    }
    if (w < 0 || b1 < 0 || b2 < 0) return false;
    const std::int64_t elements = extent_of(k, e), nq = extent_of(k, q), ni = extent_of(k, i), nj = extent_of(k, j);
    if (elements < 32 || !acro_b200_rank1_gemm_supported(static_cast<int>(nq), static_cast<int>(ni), static_cast<int>(nj))) return false;
    s = Step();
    s.family = Family::Rank1Gemm;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    s.rows = elements;
    s.sizes[0] = static_cast<int>(nq);
    s.sizes[1] = static_cast<int>(ni);
    s.sizes[2] = static_cast<int>(nj);
    for (int vari : {w, b1, b2})
    {
        TensorRef r;
        r.ki = ki;
        r.vari = vari;
        s.ins.push_back(r);
    }
    s.bytes = io_bytes(k);
    s.flops = 2 * elements * nq * ni * nj;   // GEMM form
    std::ostringstream note;
    note << "GEMM view [" << elements << " x " << nq << "] x [" << nq << " x " << ni * nj
         << "], right operand formed on the fly, fp64 tensor cores (mma.sync m8n8k4)";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- invariant_gemm
// Out_e_X = (product of batch-invariant inputs) In_e_Q: exactly one input carries the batch index e, in
// front, and its other indices are exactly the contracted ones.  The invariant inputs are multiplied
// out into P[Q x X] by the generic kernel (left to right, as written), then Out[e, X] = sum_Q In[e, Q] P[Q, X]
// is one GEMM with the batch as its row dimension.
bool plan_invariant_gemm(DimensionedKernel &k, int ki, Step &s)
{
    const Names out = k.OutputVar.IndexNames;
    const int n_in = k.GetNumInputVars();
    if (out.size() < 2 || !distinct(out) || n_in < 2 || n_in > ACRO_B200_MAX_INPUTS || k.ContractionIndexNames.empty()) return false;
    const std::string e = out[0];
    int batched = -1;
    for (int vari = 0; vari < n_in; ++vari)
    {
        const Names idx = indices_of(k, vari);
        const bool has_e = std::find(idx.begin(), idx.end(), e) != idx.end();
        if (!has_e) continue;
        if (batched >= 0 || idx[0] != e || !distinct(idx)) return false;
        batched = vari;
    }
    if (batched < 0) return false;
    const Names q_full = indices_of(k, batched);
    const Names q(q_full.begin() + 1, q_full.end());
    Names contracted = k.ContractionIndexNames, q_sorted = q;
    std::sort(contracted.begin(), contracted.end());
    std::sort(q_sorted.begin(), q_sorted.end());
    if (q_sorted != contracted) return false;
    const Names x(out.begin() + 1, out.end());
    if (q.size() + x.size() > ACRO_B200_MAX_LOOPS) return false;

    const std::int64_t elements = extent_of(k, e);
    std::int64_t kk = 1, nn = 1;
    for (const std::string &idx : q) kk *= extent_of(k, idx);
    for (const std::string &idx : x) nn *= extent_of(k, idx);
    // worth a tensor-core GEMM, and P small enough to rebuild on every call
    if (elements < 64 || nn < 16 || kk < 4 || kk * nn > (std::int64_t(1) << 26)) return false;
    if (elements * nn * kk < (std::int64_t(1) << 22)) return false;

    s = Step();
    s.family = Family::InvariantGemm;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    s.rows = elements;
    s.sizes[0] = static_cast<int>(kk);
    s.sizes[1] = static_cast<int>(nn);

    // P[q..., x...] = product of the invariant inputs, in the order they are written
    Names loops = concat(q, x);
    acro_b200_generic_desc &g = s.generic;
    std::memset(&g, 0, sizeof g);
    g.n_loops = g.n_outer = static_cast<int>(loops.size());
    g.n_inputs = n_in - 1;
    g.op = ACRO_B200_OP_ASSIGN;
    // rows of P padded to an even length: every row then starts on a 16-byte boundary
    const std::int64_t ldp = nn + (nn & 1);
    s.sizes[2] = static_cast<int>(ldp);
    std::int64_t stride = 1;
    for (int l = g.n_loops - 1; l >= 0; --l)
    {
        g.extent[l] = extent_of(k, loops[l]);
        g.out_step[l] = stride;
        stride *= g.extent[l];
        if (l == static_cast<int>(q.size())) stride = ldp;      // the first output index closes a row of P
    }
    TensorRef br;
    br.ki = ki;
    br.vari = batched;
    s.ins.push_back(br);
    int slot = 0;
    for (int vari = 0; vari < n_in; ++vari)
    {
        if (vari == batched) continue;
        const Names idx = indices_of(k, vari);
        for (int d = 0; d < static_cast<int>(idx.size()); ++d)
        {
            const int l = static_cast<int>(std::find(loops.begin(), loops.end(), idx[d]) - loops.begin());
            g.in_step[slot][l] += k.GetVarDimStride64(vari, d);
        }
        TensorRef r;
        r.ki = ki;
        r.vari = vari;
        s.ins.push_back(r);
        ++slot;
    }
    s.bytes = io_bytes(k);
    s.flops = 2 * elements * kk * nn;   // GEMM form
    std::ostringstream note;
    note << "batch-invariant inputs multiplied out into P[" << kk << " x " << nn << "], then GEMM [" << elements << " x " << kk
         << "] x P on the fp64 tensor cores (mma.sync m8n8k4)";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- batched_gemm
// C_e_i_j = A_e_i_k B_e_k_j (either operand order).
bool plan_batched_gemm(DimensionedKernel &k, int ki, Step &s)
{
    const Names out = k.OutputVar.IndexNames;
    if ((out.size() != 3 && out.size() != 2) || !distinct(out) || k.ContractionIndexNames.size() != 1 || k.GetNumInputVars() != 2) return false;
    const std::string e = out[0], kk = k.ContractionIndexNames[0];
    int av = -1, bv = -1, ta = 0, tb = 0;
    std::int64_t m = 1, n = 1;
    if (out.size() == 3)
    {
        // the input that carries i is A (stored i x k, or k x i: transposed), the one that carries j is B (k x j, or j x k)
        const std::string i = out[1], j = out[2];
        for (int vari = 0; vari < 2; ++vari)
        {
            const Names idx = indices_of(k, vari);
            if (idx == Names{e, i, kk} && av < 0) av = vari;
            else if (idx == Names{e, kk, i} && av < 0) { av = vari; ta = 1; }
            else if (idx == Names{e, kk, j} && bv < 0) bv = vari;
            else if (idx == Names{e, j, kk} && bv < 0) { bv = vari; tb = 1; }
            else return false;
        }
        m = extent_of(k, i);
        n = extent_of(k, j);
    }
    else
    {
        // element matrix times element vector, Y_e_i = M_e_i_k X_e_k (n = 1), or vector times matrix, Y_e_j = X_e_k M_e_k_j (m = 1)
        const std::string x = out[1];
        for (int vari = 0; vari < 2; ++vari)
        {
            const Names idx = indices_of(k, vari);
            if (idx == Names{e, kk}) continue;
            if (idx == Names{e, x, kk} && av < 0) av = vari;
            else if (idx == Names{e, kk, x} && bv < 0) bv = vari;
            else return false;
        }
        if ((av < 0) == (bv < 0)) return false;          // exactly one of the two is the matrix
        const int vec = av >= 0 ? 1 - av : 1 - bv;
        if (indices_of(k, vec) != Names{e, kk}) return false;
        if (av >= 0)
        {
            bv = vec;
            m = extent_of(k, x);
        }
        else
        {
            av = vec;
            n = extent_of(k, x);
        }
    }
    if (av < 0 || bv < 0) return false;
    const std::int64_t batch = extent_of(k, e), kn = extent_of(k, kk);
    if (m == 1) ta = 0;      // a row or a column is stored the same way in both orders
    if (n == 1) tb = 0;
    if (!acro_b200_batched_gemm_t_supported(static_cast<int>(m), static_cast<int>(n), static_cast<int>(kn), ta, tb)) return false;
    s = Step();
    s.family = Family::BatchedGemm;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    s.rows = batch;
    s.sizes[0] = static_cast<int>(m);
    s.sizes[1] = static_cast<int>(n);
    s.sizes[2] = static_cast<int>(kn);
    s.sizes[3] = ta;
    s.sizes[4] = tb;
    TensorRef a, b;
    a.ki = b.ki = ki;
    a.vari = av;
    b.vari = bv;
    s.ins = {a, b};
    s.bytes = io_bytes(k);
    s.flops = 2 * batch * m * n * kn;
    std::ostringstream note;
    note << batch << " products of " << m << "x" << kn << " by " << kn << "x" << n;
    if (ta) note << " (first operand stored transposed)";
    if (tb) note << " (second operand stored transposed)";
    if (m == 1 || n == 1) note << ", matrix-vector: streaming tiles of elements through shared memory (bulk copies), rows rotated across banks";
    else if (m <= 16 && n <= 16 && kn <= 16) note << ", streaming tiles of matrices through shared memory (bulk copies), 4x1 strips per thread, no fused multiply-add";
    else if (acro_b200_batched_gemm_by_pairs(static_cast<int>(m), static_cast<int>(n), static_cast<int>(kn), ta, tb))
        note << ", rows of an odd length: pairs of elements by bulk copy into unpadded slots, fp64 tensor cores (mma.sync m8n8k4); operands off a 16-byte boundary take the zero-padded ring";
    else if (!ta && !tb && (m > 32 || n > 32 || kn > 32) && !(m == 64 && n == 64 && kn == 64)) note << ", 64x64 tiles of every product through the tensor-core GEMM (mma.sync m8n8k4)";
    else
    {
        note << ", persistent CTAs, 3-stage asynchronous bulk-copy ring, fp64 tensor cores (mma.sync m8n8k4)";
        if (!(m == n && n == kn && (m == 32 || m == 64))) note << ", zero-padded on chip to " << ((m > 32 || n > 32 || kn > 32) ? 64 : 32);
    }
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- gram
// S_a_b (op)= X_n_a Y_n_b: two row operands contracted over their common leading index (X and Y may be the
// same tensor).  Rows enough to fill the machine; shorter contractions stay on the generic kernel.
bool plan_gram(DimensionedKernel &k, int ki, Step &s)
{
    const Names out = k.OutputVar.IndexNames;
    if (out.size() != 2 || !distinct(out) || k.ContractionIndexNames.size() != 1 || k.GetNumInputVars() != 2) return false;
    const std::string n = k.ContractionIndexNames[0];
    int xv = -1, yv = -1;
    for (int vari = 0; vari < 2; ++vari)
    {
        const Names idx = indices_of(k, vari);
        if (idx == Names{n, out[0]} && xv < 0) xv = vari;
        else if (idx == Names{n, out[1]} && yv < 0) yv = vari;
        else return false;
    }
    if (xv < 0 || yv < 0) return false;
    const std::int64_t rows = extent_of(k, n), a = extent_of(k, out[0]), b = extent_of(k, out[1]);
    if (a > 64 || b > 64 || !acro_b200_gram_supported(static_cast<int>(a), static_cast<int>(b))) return false;
    if (rows < 4096 || rows * a * b < (std::int64_t(1) << 20)) return false;
    s = Step();
    s.family = Family::Gram;
    s.kernels = {ki};
    s.out.ki = ki;
    s.op = op_code(k);
    s.rows = rows;
    s.sizes[0] = static_cast<int>(a);
    s.sizes[1] = static_cast<int>(b);
    TensorRef x, y;
    x.ki = y.ki = ki;
    x.vari = xv;
    y.vari = yv;
    s.ins = {x, y};
    s.bytes = rows * 8 * (a + b) + a * b * 8;
    s.flops = 2 * rows * a * b;
    std::ostringstream note;
    note << "Gram form over " << rows << " rows: ";
    if (a <= 16 && b <= 16) note << "tiles of rows streamed through shared memory (bulk copies), 4x4 blocks of the " << a << "x" << b << " result in registers";
    else note << "slabs of " << ((a > 32 || b > 32) ? 64 : 32) << " rows as " << a << "x" << b << " products on the fp64 tensor cores (mma.sync m8n8k4)";
    note << ", summed per CTA, partial tiles combined in a fixed order";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- sumfact_mass
// A kernel group is recognised by its shape, not by its names: variables and indices are
// renamed in order of first appearance and the result is compared with the same renaming of
// the sum-factorised mass operator chain.
std::string canonical_form(const std::vector<DimensionedKernel *> &kernels)
{
    std::vector<std::string> vars, idxs;
    auto id_of = [](std::vector<std::string> &table, const std::string &name) {
        auto it = std::find(table.begin(), table.end(), name);
        if (it == table.end())
        {
            table.push_back(name);
            return table.size() - 1;
        }
        return static_cast<std::size_t>(it - table.begin());
    };
    std::ostringstream os;
    for (DimensionedKernel *k : kernels)
    {
        for (int vari = -1; vari < k->GetNumInputVars(); ++vari)
        {
            os << "V" << id_of(vars, k->GetVarName(vari));
            for (const std::string &idx : indices_of(*k, vari)) os << "_x" << id_of(idxs, idx);
            if (vari < 0) os << k->EqOperator;
            else os << " ";
        }
        os << ";";
    }
    return os.str();
}

const char *const kMassChain[6] = {
    "T1_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3",  "T2_e_i1_k2_k3 = B_k2_i2 T1_e_i1_i2_k3", "X_e_k1_k2_k3 = B_k1_i1 T2_e_i1_k2_k3 W_e_k1_k2_k3",
    "Y1_e_i1_k2_k3 = B_k1_i1 X_e_k1_k2_k3", "Y2_e_i1_i2_k3 = B_k2_i2 Y1_e_i1_k2_k3", "V_e_i1_i2_i3 = B_k3_i3 Y2_e_i1_i2_k3"};

std::string canonical_text_form(const char *const *texts, int n)
{
    // Same renaming applied to plain strings (the pattern has no tensors attached).
    std::vector<std::string> vars, idxs;
    auto id_of = [](std::vector<std::string> &table, const std::string &name) {
        auto it = std::find(table.begin(), table.end(), name);
        if (it == table.end())
        {
            table.push_back(name);
            return table.size() - 1;
        }
        return static_cast<std::size_t>(it - table.begin());
    };
    std::ostringstream os;
    for (int i = 0; i < n; ++i)
    {
        TensorKernel k(texts[i]);
        for (int vari = -1; vari < k.GetNumInputVars(); ++vari)
        {
            os << "V" << id_of(vars, k.GetVarName(vari));
            const Names &names = vari < 0 ? k.OutputVar.IndexNames : k.InputVars[vari].IndexNames;
            for (const std::string &idx : names) os << "_x" << id_of(idxs, idx);
            if (vari < 0) os << k.EqOperator;
            else os << " ";
        }
        os << ";";
    }
    return os.str();
}

bool plan_sumfact_mass(DimensionedMultiKernel &mk, Step &s)
{
    if (mk.GetNumKernels() != 6) return false;
    static const std::string pattern = canonical_text_form(kMassChain, 6);
    if (canonical_form(mk.Kernels) != pattern) return false;
    DimensionedKernel &first = *mk.Kernels[0];   // T1_e_i1_i2_k3 = B_k3_i3 U_e_i1_i2_i3
    DimensionedKernel &third = *mk.Kernels[2];   // X_e_k1_k2_k3 = B_k1_i1 T2_e_i1_k2_k3 W_e_k1_k2_k3
    const Names u = indices_of(first, 1), x = indices_of(third, -1);
    const std::int64_t elements = extent_of(first, u[0]);
    const std::int64_t p = extent_of(first, u[1]), q = extent_of(third, x[1]);
    for (int d = 1; d < 4; ++d)
    {
        if (extent_of(first, u[d]) != p || extent_of(third, x[d]) != q) return false;
    }
    if (!acro_b200_sumfact_mass_supported(static_cast<int>(p), static_cast<int>(q))) return false;

    s = Step();
    s.family = Family::SumfactMass;
    s.kernels = {0, 1, 2, 3, 4, 5};
    s.op = ACRO_B200_OP_ASSIGN;
    s.rows = elements;
    s.sizes[0] = static_cast<int>(p);
    s.sizes[1] = static_cast<int>(q);
    s.out.ki = 5;                       // V
    TensorRef b, uu, w;
    b.ki = 0; b.vari = 0;               // B
    uu.ki = 0; uu.vari = 1;             // U
    w.ki = 2; w.vari = 2;               // W
    s.ins = {b, uu, w};
    for (int ki = 0; ki < 5; ++ki)
    {
        TensorRef r;
        r.ki = ki;
        s.elided.push_back(r);
    }
    s.bytes = elements * 8 * (2 * p * p * p + q * q * q) + 8 * p * q;
    // as written: one multiply-add per term of every stage, plus the extra factor W in stage three
    s.flops = elements * (2 * (p * p * q * p + p * q * q * p + q * q * q * p + p * q * q * q + p * p * q * q + p * p * p * q) + q * q * q * p);
    std::ostringstream note;
    note << "six stages fused, " << elements << " elements, p=" << p << " q=" << q
         << "; intermediates in registers/shared memory, operands by asynchronous bulk copy";
    s.note = note.str();
    return true;
}

// ---------------------------------------------------------------- permute
// Out = In with the indices in another order, fastest index included: a tiled transpose.
bool plan_permute(DimensionedKernel &k, int ki, Step &s)
{
    if (k.GetNumInputVars() != 1 || !k.ContractionIndexNames.empty()) return false;
    const Names out = k.OutputVar.IndexNames, in = indices_of(k, 0);
    if (out.size() != in.size() || !distinct(out) || !distinct(in)) return false;
    Step g = plan_generic(k, ki);
    if (!acro_b200_permute_supported(&g.generic)) return false;
    // both fastest indices long enough to fill a good part of the 64 x 64 tiles, and enough data to matter
    std::int64_t ext_fo = 0, ext_fi = 0, total = 1;
    for (int l = 0; l < g.generic.n_loops; ++l)
    {
        total *= g.generic.extent[l];
        if (g.generic.out_step[l] == 1 && g.generic.extent[l] > 1) ext_fo = g.generic.extent[l];
        if (g.generic.in_step[0][l] == 1 && g.generic.extent[l] > 1) ext_fi = g.generic.extent[l];
    }
    if (ext_fo < 16 || ext_fi < 16 || total < (std::int64_t(1) << 16)) return false;
    s = g;
    s.family = Family::Permute;
    s.zero_fill_first = false;
    std::ostringstream note;
    note << "tiled transpose: 64x64 tiles over the fastest output index (" << ext_fo << ") and the fastest input index (" << ext_fi
         << "), " << total << " entries";
    s.note = note.str();
    return true;
}

Step plan_family(DimensionedKernel &k, int ki)
{
    Step s;
    // debugging aid: ACRO_B200_ONLY_GENERIC=1 in the environment plans every kernel on the generic family
    const char *only_generic = std::getenv("ACRO_B200_ONLY_GENERIC");
    if (only_generic != nullptr && only_generic[0] == '1') return plan_generic(k, ki);
    if (plan_reduce_batch(k, ki, s)) return s;
    if (plan_pointwise_sym(k, ki, s)) return s;
    if (plan_rank1_gemm(k, ki, s)) return s;
    if (plan_batched_gemm(k, ki, s)) return s;
    if (plan_permute(k, ki, s)) return s;
    if (plan_gram(k, ki, s)) return s;
    if (plan_invariant_gemm(k, ki, s)) return s;
    return plan_generic(k, ki);
}

Step plan_single(DimensionedKernel &k, int ki)
{
    Step s = plan_family(k, ki);
    // Whatever family runs it: which inputs would, as a rank's slab, leave this rank with a partial sum only?
    for (int vari = 0; vari < k.GetNumInputVars(); ++vari)
    {
        const Names idx = indices_of(k, vari);
        if (idx.empty()) continue;
        if (std::find(k.ContractionIndexNames.begin(), k.ContractionIndexNames.end(), idx[0]) == k.ContractionIndexNames.end()) continue;
        TensorRef r;
        r.ki = ki;
        r.vari = vari;
        s.lead_contracted.push_back(r);
    }
    return s;
}

}  // namespace

const char *FamilyName(Family f)
{
    switch (f)
    {
        case Family::Generic: return "generic";
        case Family::ReduceBatch: return "reduce_batch";
        case Family::PointwiseSym: return "pointwise_sym";
        case Family::Rank1Gemm: return "rank1_gemm";
        case Family::BatchedGemm: return "batched_gemm";
        case Family::SumfactMass: return "sumfact_mass";
        case Family::InvariantGemm: return "invariant_gemm";
        case Family::Permute: return "permute";
        case Family::Gram: return "gram";
    }
    return "?";
}

Program BuildProgram(DimensionedMultiKernel &mk, bool allow_elision)
{
    Program p;
    if (allow_elision)
    {
        Step fused;
        if (plan_sumfact_mass(mk, fused))
        {
            p.steps.push_back(fused);
            p.elides = true;
            return p;
        }
    }
    for (int ki = 0; ki < mk.GetNumKernels(); ++ki)
    {
        p.steps.push_back(plan_single(*mk.Kernels[ki], ki));
    }
    for (const Step &s : p.steps)
    {
        if (s.family == Family::ReduceBatch)
        {
            p.scratch_bytes = std::max(p.scratch_bytes, acro_b200_reduce_batch_scratch_bytes(s.sizes[0]));
        }
        if (s.family == Family::Generic)
        {
            p.scratch_bytes = std::max(p.scratch_bytes, acro_b200_generic_scratch_bytes(&s.generic));
        }
        if (s.family == Family::Gram)
        {
            p.scratch_bytes = std::max(p.scratch_bytes, acro_b200_gram_scratch_bytes(s.sizes[0], s.sizes[1]));
        }
        if (s.family == Family::InvariantGemm)
        {
            p.scratch_bytes = std::max(p.scratch_bytes, static_cast<std::size_t>(s.sizes[0]) * static_cast<std::size_t>(s.sizes[2]) * sizeof(double));
        }
    }
    return p;
}

std::string Program::Describe(DimensionedMultiKernel &mk) const
{
    std::ostringstream os;
    os << "acrotensor-b200 plan (sm_100a, ahead-of-time kernels)\n";
    os << "kernels:";
    for (DimensionedKernel *k : mk.Kernels) os << " [" << k->KernelStr << "]";
    os << "\nloop order:";
    for (int l = 0; l < mk.GetNumIndices(); ++l)
    {
        os << " " << mk.GetLoopIndex(l) << "(" << mk.GetLoopDim(l) << ")" << (mk.IsContractionLoop(l) ? "*" : "")
           << (mk.IsSharedOuterLoop(l) ? "^" : "");
    }
    os << "   (* contracted, ^ shared outer)\n";
    os << "unique variables: " << mk.GetNumUVars() << "\n";
    for (std::size_t i = 0; i < steps.size(); ++i)
    {
        const Step &s = steps[i];
        os << "step " << i << ": family=" << FamilyName(s.family) << " kernels=";
        for (std::size_t j = 0; j < s.kernels.size(); ++j) os << (j ? "," : "") << s.kernels[j];
        os << " bytes=" << s.bytes << " flops=" << s.flops << " | " << s.note << "\n";
        if (!s.lead_contracted.empty())
        {
            os << "        summed over the ranks of a peer group when one of these inputs is a rank's slab:";
            for (const TensorRef &r : s.lead_contracted) os << " " << mk.Kernels[r.ki]->GetVarName(r.vari);
            os << (s.family == Family::ReduceBatch ? " (all-reduce fused into the kernel)" : " (all-reduce kernel after the step)") << "\n";
        }
    }
    if (scratch_bytes) os << "scratch: " << scratch_bytes << " bytes\n";
    return os.str();
}

}
}
