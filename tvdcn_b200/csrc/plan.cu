// Engine choice and workspace layout.
#include "plan.h"

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
}  // namespace

Plan plan_forward(const tvdcn_problem *p) {
    Plan pl;
    pl.why_not = "tensor-core forward not built yet";
    const GeoHost g = make_geo_host(p);
    Bump b;
    if (p->transposed && is16(p->dtype)) pl.img_acc = b.take((size_t)g.B * g.Cs * g.S * sizeof(float));
    pl.total = b.off;
    return pl;
}

Plan plan_backward(const tvdcn_problem *p, bool want_input, bool want_weight, bool want_offset, bool want_mask) {
    Plan pl;
    pl.why_not = "tensor-core backward not built yet";
    const GeoHost g = make_geo_host(p);
    Bump b;
    if (is16(p->dtype)) {
        if (!p->transposed && want_input) pl.img_acc = b.take((size_t)g.B * g.Cs * g.S * sizeof(float));
        if (want_weight) pl.gw_acc = b.take((size_t)g.Cd * (g.Cs / g.groups) * g.K * sizeof(float));
    }
    if (is16(p->aux_dtype)) {
        if (want_offset && g.og > 0) pl.goff_acc = b.take((size_t)g.B * g.og * g.K * g.dim * g.P * sizeof(float));
        if (want_mask && g.mg > 0) pl.gmask_acc = b.take((size_t)g.B * g.mg * g.K * g.P * sizeof(float));
    }
    pl.total = b.off;
    return pl;
}

int tensor_forward(const tvdcn_problem *, const GeoHost &, const Plan &, const void *, const void *, const void *,
                   const void *, const void *, void *, char *, cudaStream_t) {
    return fail(TVDCN_ERR_UNSUPPORTED, "tensor-core forward not built");
}

int tensor_backward(const tvdcn_problem *, const GeoHost &, const Plan &, const void *, const void *, const void *,
                    const void *, const void *, void *, void *, void *, void *, void *, char *, cudaStream_t) {
    return fail(TVDCN_ERR_UNSUPPORTED, "tensor-core backward not built");
}

}  // namespace tvdcn_b200
