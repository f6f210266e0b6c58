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
    // .int(8) over a lone Q6_K tensor: recipe re-encodes it to Q8_0 at load (finish_int_sums, recipe.rs:22345-22369), and so does place()
    {
        std::vector<uint8_t> b8((size_t)hidden * mid / 32 * 34);
        rqo_requantize_q8_0(RQO_Q6_K, b2.data(), (int64_t)hidden * mid, b8.data(), 4);
        std::vector<float> xin2(mid), ref8(hidden);
        rqo_normal(73, 0, 0, mid, 1.0, xin2.data());
        rqo_matvec(RQO_Q8_0, b8.data(), hidden, mid, xin2.data(), 1, 1, ref8.data(), 1, RQO_ACT_INT8, 32, 4);
        auto lone = Model().layer({RQ_Q6_K, hidden, mid, b2.data()}).int_(8).place(0);
        std::vector<double> y8 = lone.infer(std::vector<double>(xin2.begin(), xin2.end()));
        const double e3 = rel_err(y8, ref8);
        if (!(e3 <= 5e-5)) { std::printf("lone Q6_K under int(8): relative error %g against the Q8_0 re-encode\n", e3); return 1; }
        if (lone.resident_bytes()[0] != b8.size()) { std::printf("re-encoded weight holds %zu bytes, expected %zu\n", lone.resident_bytes()[0], b8.size()); return 1; }
    }
    // .int(4): storage Q4_1 by the load kernel's encoder, int8 records against its codes (recipe.rs:22348); place() re-encodes
    {
        std::vector<uint8_t> b4((size_t)mid * hidden / 32 * 20);
        rqo_requantize_q4_1(RQO_Q4_K, b1.data(), (int64_t)mid * hidden, b4.data(), 4);
        std::vector<float> xin4(hidden), ref4(mid);
        rqo_normal(75, 0, 0, hidden, 1.0, xin4.data());
        rqo_matvec(RQO_Q4_1, b4.data(), mid, hidden, xin4.data(), 1, 1, ref4.data(), 1, RQO_ACT_INT8, 32, 4);
        auto four = Model().layer({RQ_Q4_K, mid, hidden, b1.data()}).int_(4).place(0);
        std::vector<double> y4 = four.infer(std::vector<double>(xin4.begin(), xin4.end()));
        const double e4 = rel_err(y4, ref4);
        if (!(e4 <= 5e-4)) { std::printf("Q4_K under int(4): relative error %g against the Q4_1 re-encode\n", e4); return 1; }
        if (four.resident_bytes()[0] != b4.size()) { std::printf("Q4_1 weight holds %zu bytes, expected %zu\n", four.resident_bytes()[0], b4.size()); return 1; }
        try { Model().layer({RQ_Q4_K, mid, hidden, b1.data()}).int_(16); std::printf("int(16) accepted\n"); return 1; } catch (const RecipeError&) {}
    }
    // ids -> embedding -> two layers: prefill, step and greedy decode; a step gives the bits its position gets in a prefill
    {
        const int vocab = 96;
        std::vector<float> emb((size_t)vocab * hidden), head((size_t)vocab * hidden);
        rqo_normal(74, 0, 0, (int64_t)emb.size(), 1.0, emb.data());
        rqo_normal(74, 1, 0, (int64_t)head.size(), 0.02, head.data());
        std::vector<uint8_t> be(emb.size() / 32 * 34), bh(head.size() / 256 * 144);
        rqo_quantize(RQO_Q8_0, emb.data(), (int64_t)emb.size(), be.data(), 4);
        rqo_quantize(RQO_Q4_K, head.data(), (int64_t)head.size(), bh.data(), 4);
        auto lm = Model().embed({RQ_Q8_0, vocab, hidden, be.data()}).layer({RQ_Q4_K, mid, hidden, b1.data()}).int_(8).layer({RQ_Q6_K, hidden, mid, b2.data()}).fp(32)
                      .layer({RQ_Q4_K, vocab, hidden, bh.data()}).fp(32).place(0);
        const std::vector<uint32_t> prompt = {5, 17, 3, 90, 41};
        std::vector<double> whole = lm.prefill(prompt);
        std::vector<double> part = lm.prefill({5, 17, 3, 90});
        std::vector<double> stepped = lm.step(41);
        if (whole != stepped) { std::printf("a step differs from the same position of a prefill\n"); return 1; }
        if (lm.ids() != prompt) { std::printf("the retained prefix is wrong\n"); return 1; }
        // the last position against the oracle: embedding row, then the three layers
        std::vector<float> row(hidden), h1(mid), h2(hidden), lg(vocab);
        std::vector<float> table((size_t)vocab * hidden);
        rqo_dequantize(RQO_Q8_0, be.data(), (int64_t)table.size(), table.data(), 4);
        for (int k = 0; k < hidden; ++k) row[k] = table[(size_t)41 * hidden + k];
        rqo_matvec(RQO_Q4_K, b1.data(), mid, hidden, row.data(), 1, 1, h1.data(), 1, RQO_ACT_INT8, 32, 4);
        rqo_matvec(RQO_Q6_K, b2.data(), hidden, mid, h1.data(), 1, 1, h2.data(), 1, RQO_ACT_FLOAT_RUN, 32, 4);
        rqo_matvec(RQO_Q4_K, bh.data(), vocab, hidden, h2.data(), 1, 1, lg.data(), 1, RQO_ACT_FLOAT_RUN, 32, 4);
        const double e4 = rel_err(whole, lg);
        if (!(e4 <= 1e-3)) { std::printf("prefill logits relative error %g\n", e4); return 1; }
        std::vector<uint32_t> gen = lm.decode(prompt, {7}, 4);
        if (gen.empty() || gen.size() > 4) { std::printf("decode produced %zu ids\n", gen.size()); return 1; }
        uint32_t best = 0;
        for (int i = 1; i < vocab; ++i) if (lg[i] > lg[best]) best = (uint32_t)i;
        if (gen[0] != best) { std::printf("greedy decode picked %u, the oracle's largest logit is %u\n", gen[0], best); return 1; }
        try { lm.infer(std::vector<double>(hidden, 0.0)); std::printf("infer accepted a model of ids\n"); return 1; } catch (const RecipeError&) {}
        try { lm.prefill({1000}); std::printf("an id outside the table was accepted\n"); return 1; } catch (const RecipeError&) {}
        lm.clear();
        try { lm.step(1); std::printf("step without a prefill was accepted\n"); return 1; } catch (const RecipeError& e) {
            if (std::string(e.what()) != "step requires a completed prefill") { std::printf("wrong text: %s\n", e.what()); return 1; }
        }
    }
    std::printf("ok %g %g\n", e1, e2);
    return 0;
}
