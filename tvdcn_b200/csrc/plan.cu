// Engine choice per GEMM-shaped primitive and workspace layout.
#include "plan.h"

#include <algorithm>

namespace tvdcn_b200 {

namespace {
struct Bump {
    size_t off = 0;
    size_t take(size_t bytes) {
        const size_t at = off;
        off = align_up(off + bytes);
        return at;
    }
};
bool is16(int dt) { return dt == DT_F16 || dt == DT_BF16; }

// Shape conditions shared by all tensor-core kernels: K chunks of 64 channels of one tap must not
// straddle a convolution, offset or mask group, and rows of the channels-last image are indexed in 32 bits.
const char *tc_common(const tvdcn_problem *p, const GeoHost &g) {
    if (p->engine == TVDCN_ENGINE_SIMT) return "SIMT engine requested";
    if (p->dtype == TVDCN_F64) return "f64 has no tensor-core kind";
    if (p->aux_dtype != TVDCN_F32) return "offset / mask / bias must be f32 for the tensor-core kernels";
    const int csg = g.Cs / g.groups, cdg = g.Cd / g.groups;
    if (csg % 64 != 0) return "sampled channels per group must be a multiple of 64";
    if (cdg % 64 != 0) return "dense channels per group must be a multiple of 64";
    if (g.K > 512) return "more than 512 kernel taps (the tensor-core kernels tabulate tap coordinates)";
    if (g.B > 65535) return "batch above 65535 (the layout staging kernels put the batch in gridDim.z)";
    if (g.og > 0 && (g.Cs / g.og) % 64 != 0) return "channels per offset group must be a multiple of 64";
    if (g.mg > 0 && (g.Cs / g.mg) % 64 != 0) return "channels per mask group must be a multiple of 64";
    if (((long long)g.B * g.S + 1) * g.Cs >= (1LL << 31) || (long long)g.B * g.P >= (1LL << 31))
        return "sampled image has 2^31 elements or more (32-bit element offsets)";
    if ((long long)g.Cd * csg * g.K >= (1LL << 31)) return "weight has 2^31 elements or more (32-bit packing indices)";
    return nullptr;
}

// f32 data on the tensor cores: one accumulator may take about 2400 MMAs before the round-toward-zero error of
// the f32 accumulation (~2e-8 of the result per MMA) eats half of the 1e-4 budget.  The sample -> GEMM kernel adds
// 12 MMAs per (tap, 64-channel chunk), spread over min(4, 512 / bn) accumulators.
bool chain_ok(int mode, const GeoHost &g, int bn) {
    if (mode != 2) return true;
    const int nacc = std::min(4, 512 / std::max(bn, 1));
    const long long chain = (long long)g.K * (g.Cs / g.groups / 64) * 12 / nacc;
    return chain <= 2400;
}

// buffers of the GEMM -> scatter kernel
void take_scatter_buffers(Plan &pl, Bump &b, const tvdcn_problem *p, const GeoHost &g, bool scatter) {
    const size_t nw = (size_t)g.Cd * (g.Cs / g.groups) * g.K;
    pl.w_pack_kd = b.take(nw * 2);
    if (p->dtype == TVDCN_F32) pl.w_pack_kd_lo = b.take(nw * 2);
    if (scatter) pl.img_grad_cl = b.take((size_t)g.B * g.S * g.Cs * sizeof(float));
}
}  // namespace

int tc_mode_of(int dtype) { return dtype == DT_F32 ? 2 : (dtype == DT_F16 ? 1 : 0); }

Plan plan_forward(const tvdcn_problem *p) {
    Plan pl;
    const GeoHost g = make_geo_host(p);
    Bump b;
    const char *why = tc_common(p, g);
    const int mode = tc_mode_of(p->dtype);
    const size_t es = p->dtype == TVDCN_F32 ? 4 : 2;
    const size_t nw = (size_t)g.Cd * (g.Cs / g.groups) * g.K;
    int bn = 0, st = 0, gbufs = 0;
    if (why == nullptr && !p->transposed) {
        if (fwd_tc_config(g.dim, mode, g.Cd / g.groups, &bn, &st) && chain_ok(mode, g, bn)) {
            pl.tensor = pl.tc_sg = true;
            pl.img_cl = b.take(((size_t)g.B * g.S + 1) * g.Cs * es);   // + one row of zeros, see stage_image
            pl.w_pack = b.take(nw * 2);
            if (p->dtype == TVDCN_F32) pl.w_pack_lo = b.take(nw * 2);
        } else {
            why = "no tile configuration fits (or the f32 accumulation chain would be too long)";
        }
    } else if (why == nullptr) {
        if (dgrad_tc_config(g.dim, mode, g.Cd / g.groups, g.K, &bn, &gbufs, &st)) {
            pl.tensor = pl.tc_gs = true;
            take_scatter_buffers(pl, b, p, g, true);
        } else {
            why = "no tile configuration fits";
        }
    }
    if (why != nullptr) {
        pl.why_not = why;
        if (p->transposed && is16(p->dtype)) pl.img_acc = b.take((size_t)g.B * g.Cs * g.S * sizeof(float));
    }
    pl.total = b.off;
    return pl;
}

Plan plan_backward(const tvdcn_problem *p, bool want_input, bool want_weight, bool want_offset, bool want_mask) {
    Plan pl;
    const GeoHost g = make_geo_host(p);
    Bump b;
    const char *why = tc_common(p, g);
    const int mode = tc_mode_of(p->dtype);
    const size_t es = p->dtype == TVDCN_F32 ? 4 : 2;
    const size_t nw = (size_t)g.Cd * (g.Cs / g.groups) * g.K;
    want_offset = want_offset && g.og > 0;
    want_mask = want_mask && g.mg > 0;
    if (why == nullptr) {
        int bn = 0, st = 0, ns = 0, mt = 0, gbufs = 0;
        // which primitives run on the tensor cores
        // transposed backward: grad_input is a sample -> GEMM over grad_output
        pl.tc_sg = p->transposed && want_input && fwd_tc_config(g.dim, mode, g.Cd / g.groups, &bn, &st) &&
                   chain_ok(mode, g, bn);
        pl.tc_sw = want_weight && wgrad_tc_config(g.dim, mode, g.Cd / g.groups, g.P, &ns, &mt, &st);
        // conv: scatter into grad_input + coordinate gradients; transposed: coordinate gradients only
        const bool scatter = !p->transposed && want_input;
        pl.tc_gs = (scatter || want_offset || want_mask) &&
                   dgrad_tc_config(g.dim, mode, g.Cd / g.groups, g.K, &bn, &gbufs, &st);
        pl.tensor = pl.tc_sg || pl.tc_sw || pl.tc_gs;
        // The staged image comes first, as in the forward plan: a backward call that is told to reuse the
        // forward call's staging (TVDCN_FLAG_REUSE_STAGED_INPUT) finds it at the same offset of the same workspace.
        if (pl.tensor) pl.img_cl = b.take(((size_t)g.B * g.S + 1) * g.Cs * es);
        if (pl.tc_sg) {
            pl.w_pack = b.take(nw * 2);
            if (p->dtype == TVDCN_F32) pl.w_pack_lo = b.take(nw * 2);
        }
        if (pl.tc_sw && p->dtype == TVDCN_F32) {
            pl.dense_hi = b.take((size_t)g.B * g.Cd * g.P * 2);
            pl.dense_lo = b.take((size_t)g.B * g.Cd * g.P * 2);
        }
        if (pl.tc_gs) take_scatter_buffers(pl, b, p, g, scatter);
        if (!pl.tensor) pl.why_not = "no tensor-core kernel covers the requested gradients for this shape";
    } else {
        pl.why_not = why;
    }
    if (is16(p->dtype)) {
        if (!p->transposed && want_input && !pl.tc_gs) pl.img_acc = b.take((size_t)g.B * g.Cs * g.S * sizeof(float));
    }
    // 16-bit data accumulates the weight gradient in f32; the tensor-core kernel accumulates (any data type) into
    // a staged layout that a small kernel turns into the caller's afterwards
    if (want_weight && (is16(p->dtype) || pl.tc_sw)) pl.gw_acc = b.take(nw * sizeof(float));
    if (is16(p->aux_dtype)) {
        if (want_offset) pl.goff_acc = b.take((size_t)g.B * g.og * g.K * g.dim * g.P * sizeof(float));
        if (want_mask) pl.gmask_acc = b.take((size_t)g.B * g.mg * g.K * g.P * sizeof(float));
    }
    pl.total = b.off;
    return pl;
}

}  // namespace tvdcn_b200
