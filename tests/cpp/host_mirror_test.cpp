// The C++ host mirror (include/recipe_rq.hpp) against the CPU oracle: a chain of two quantised
// layers under .int(8) and .fp(32), then a gguf_moe block, through Placed::infer.
// Built and run by tests/test_gpu_host_mirror.py. Prints "ok" on success.
#include <cmath>
#include <cstdio>
#include <vector>

#include "recipe_rq.hpp"
extern "C" {
#include "rq_oracle.h"
}

static double rel_err(const std::vector<double>& y, const std::vector<float>& ref) {
    double peak = 0, worst = 0;
    for (float r : ref) peak = std::fmax(peak, std::fabs(r));
    for (size_t i = 0; i < ref.size(); ++i) worst = std::fmax(worst, std::fabs(y[i] - ref[i]) / std::fmax(std::fabs(ref[i]), 1e-3 * peak));
    return worst;
}

int main() {
    using namespace recipe;
    const int hidden = 512, mid = 768;
    std::vector<float> w1((size_t)mid * hidden), w2((size_t)hidden * mid), x(hidden);
    rqo_normal(71, 0, 0, (int64_t)w1.size(), 0.02, w1.data());
    rqo_normal(71, 1, 0, (int64_t)w2.size(), 0.02, w2.data());
    rqo_normal(71, 2, 0, hidden, 1.0, x.data());
    std::vector<uint8_t> b1(w1.size() / 256 * 144), b2(w2.size() / 256 * 210);
    rqo_quantize(RQO_Q4_K, w1.data(), (int64_t)w1.size(), b1.data(), 4);
    rqo_quantize(RQO_Q6_K, w2.data(), (int64_t)w2.size(), b2.data(), 4);
    // recipe.model().layer(w1).int(8).layer(w2).fp(32)
    Model model = Model().layer({RQ_Q4_K, mid, hidden, b1.data()}).int_(8).layer({RQ_Q6_K, hidden, mid, b2.data()}).fp(32);
    auto placed = model.place(0);
    std::vector<double> xin(x.begin(), x.end());
    std::vector<double> y = placed.infer(xin);
    std::vector<float> h(mid), ref(hidden);
    rqo_matvec(RQO_Q4_K, b1.data(), mid, hidden, x.data(), 1, 1, h.data(), 1, RQO_ACT_INT8, 32, 4);
    rqo_matvec(RQO_Q6_K, b2.data(), hidden, mid, h.data(), 1, 1, ref.data(), 1, RQO_ACT_FLOAT_RUN, 32, 4);
    const double e1 = rel_err(y, ref);
    if (!(e1 <= 1e-3)) { std::printf("layer chain relative error %g\n", e1); return 1; }
    if (placed.resident_bytes()[0] != b1.size() + b2.size()) { std::printf("resident bytes %zu\n", placed.resident_bytes()[0]); return 1; }
    // error behaviour: the reference panics with these texts
    try { Model().layer({RQ_Q4_K, mid, hidden, b1.data()}).int_(7); std::printf("int(7) accepted\n"); return 1; } catch (const RecipeError& e) {
        if (std::string(e.what()) != "int bits must be 4, 8, 16, or 32") { std::printf("wrong text: %s\n", e.what()); return 1; }
    }
    try { Model().layer({RQ_Q4_K, mid, 500, b1.data()}).place(0); std::printf("bad width accepted\n"); return 1; } catch (const RecipeError&) {}
    // a gguf_moe block: 8 experts, top-2, softmax, renormalised, gated shared expert
    const int experts = 8, top = 2, ffn = 256, mh = 256;
    std::vector<float> g((size_t)experts * ffn * mh), u(g.size()), d(g.size()), sg((size_t)ffn * mh), su(sg.size()), sd(sg.size()), sv(mh), xm(mh), sc(experts);
    rqo_normal(72, 0, 0, (int64_t)g.size(), 0.05, g.data()); rqo_normal(72, 1, 0, (int64_t)u.size(), 0.05, u.data()); rqo_normal(72, 2, 0, (int64_t)d.size(), 0.05, d.data());
    rqo_normal(72, 3, 0, (int64_t)sg.size(), 0.05, sg.data()); rqo_normal(72, 4, 0, (int64_t)su.size(), 0.05, su.data()); rqo_normal(72, 5, 0, (int64_t)sd.size(), 0.05, sd.data());
    rqo_normal(72, 6, 0, mh, 0.05, sv.data()); rqo_normal(72, 7, 0, mh, 1.0, xm.data()); rqo_normal(72, 8, 0, experts, 1.0, sc.data());
    auto q = [](const std::vector<float>& v) { std::vector<uint8_t> b(v.size() / 256 * 144); rqo_quantize(RQO_Q4_K, v.data(), (int64_t)v.size(), b.data(), 4); return b; };
    auto bg = q(g), bu = q(u), bd = q(d), bsg = q(sg), bsu = q(su), bsd = q(sd);
    MoeTensors mt{RQ_Q4_K, bg.data(), bu.data(), bd.data(), bsg.data(), bsu.data(), bsd.data(), sv.data()};
    auto moe = Model().gguf_moe(mt, experts, top, mh, ffn, Activation::Silu, Scoring::Softmax, true, SharedExpert::gated(1), 1.0, false).place(0);
    std::vector<double> ym = moe.infer(std::vector<double>(xm.begin(), xm.end()), std::vector<double>(sc.begin(), sc.end()));
    std::vector<float> routing(experts), yref(mh);
    rqo_topk(sc.data(), experts, 1, top, 0, 1, nullptr, routing.data());
    rqo_moe_forward(RQO_Q4_K, bg.data(), bu.data(), bd.data(), experts, top, mh, ffn, xm.data(), routing.data(), 1, bsg.data(), bsu.data(), bsd.data(), sv.data(), yref.data(), 4);
    const double e2 = rel_err(ym, yref);
    if (!(e2 <= 1e-3)) { std::printf("moe relative error %g\n", e2); return 1; }
    std::printf("ok %g %g\n", e1, e2);
    return 0;
}
