// recipe_rq.hpp -- the host side above the C ABI, in C++ (header only).
//
// The reference's host is Rust; where no Rust toolchain exists this header gives the same
// surface for the quantised matvec path: the names, argument meaning and error behaviour of
// recipe's `Block::fp/int`, `Model::layer`, `Model::gguf_moe`, `Placed::infer/clear/
// resident_bytes/moved_bytes` (recipe.rs:14027-14054, :14671, :14722, :21314-21490). As in
// recipe, host numbers are f64 at the API and become the model type (fp32) on upload
// (encode_floats, recipe.rs:2072-2075); internals report errors as RecipeError (recipe.rs:13416-13433)
// and the public methods throw it with the library's text (recipe panics with the same text).
// Every operation runs on the GPU through librq_b200.so; nothing here computes on the host.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "rq.h"

namespace recipe {

struct RecipeError : std::runtime_error {
    explicit RecipeError(const std::string& text) : std::runtime_error(text) {}
};
inline void require(int status) {
    if (status != RQ_OK) throw RecipeError(rq_last_error());
}

enum class Scoring { Softmax = RQ_SCORE_SOFTMAX, Sigmoid = RQ_SCORE_SIGMOID };  // recipe.rs:13955
enum class Activation { Silu };                                                   // the expert activation this path serves
struct SharedExpert {                                                             // recipe.rs:13855-13862
    enum Kind { None, Gated } kind = None;
    int count = 1;
    static SharedExpert none() { return {}; }
    static SharedExpert gated(int count) { return {Gated, count}; }
};

// A stored GGUF tensor as the file holds it: type, shape, host blocks.
struct Tensor {
    int ggml_type;
    int64_t rows, cols;
    const void* blocks;
};
struct MoeTensors {  // recipe.rs:14382-14420
    int ggml_type;
    const void *gate, *up, *down;                                    // [experts][ffn][hidden] x 2, [experts][hidden][ffn]
    const void *shared_gate = nullptr, *shared_up = nullptr, *shared_down = nullptr;
    const float* shared_gate_vector = nullptr;                        // [hidden]
};

// One block of the chain. `fp(32)` keeps activations as they are; `int_(8)` rounds them to int8
// records (step from the profile: 32 for `recipe`, 256 for `llamacpp`).
class Block {
  public:
    enum Kind { Layer, Moe } kind = Layer;
    Tensor tensor{};
    MoeTensors moe{};
    int experts = 0, top_k = 0, hidden = 0, ffn = 0;
    Scoring scoring = Scoring::Softmax;
    bool renormalize = true;
    SharedExpert shared{};
    double scale = 1.0;
    int act_mode = RQ_ACT_FLOAT, step = 32;

    Block fp(uint8_t bits) const {
        if (bits != 32) throw RecipeError("fp bits must be 32 on this path");
        Block b = *this;
        b.act_mode = RQ_ACT_FLOAT;
        return b;
    }
    Block int_(uint8_t bits) const {  // `int` is a keyword in C++
        if (bits != 4 && bits != 8 && bits != 16 && bits != 32) throw RecipeError("int bits must be 4, 8, 16, or 32");
        if (bits != 8) throw RecipeError("int(" + std::to_string(bits) + ") has no NVIDIA capability in recipe (recipe.rs:2658-2681); this path serves int(8)");
        if (kind == Moe) throw RecipeError("int sums are only for contractions: expert tables keep their activations (recipe.rs:22340)");
        Block b = *this;
        b.act_mode = RQ_ACT_INT8;
        return b;
    }
    Block with_step(int s) const {
        if (s != 32 && s != 256) throw RecipeError("int8 step must be 32 or 256");
        Block b = *this;
        b.step = s;
        return b;
    }
};

class Placed;

class Model {
  public:
    std::vector<Block> blocks;
    // A projection bound to a stored tensor (Model::layer, recipe.rs:14671).
    Model layer(const Tensor& t) const {
        Model m = *this;
        Block b;
        b.kind = Block::Layer;
        b.tensor = t;
        m.blocks.push_back(b);
        return m;
    }
    // Applies a precision to the block just added, as `recipe.model().layer(n).int(8)` reads.
    Model fp(uint8_t bits) const { Model m = *this; if (m.blocks.empty()) throw RecipeError("no block to set a precision on"); m.blocks.back() = m.blocks.back().fp(bits); return m; }
    Model int_(uint8_t bits) const { Model m = *this; if (m.blocks.empty()) throw RecipeError("no block to set a precision on"); m.blocks.back() = m.blocks.back().int_(bits); return m; }
    Model with_step(int s) const { Model m = *this; if (m.blocks.empty()) throw RecipeError("no block to set a step on"); m.blocks.back() = m.blocks.back().with_step(s); return m; }
    // Model::gguf_moe (recipe.rs:14722): the router scores are the block's second input.
    Model gguf_moe(const MoeTensors& t, int experts, int top_k, int hidden, int ffn, Activation, Scoring scoring, bool renormalize, SharedExpert shared, double scale,
                   bool selection_bias) const {
        if (experts == 0) throw RecipeError("moe requires an expert");
        if (top_k == 0 || top_k > experts) throw RecipeError("moe top-k is invalid");
        if (hidden == 0) throw RecipeError("moe expert width must be positive");
        if (!(scale == scale) || scale > 1e300 || scale < -1e300) throw RecipeError("moe routed scale must be finite");
        if (selection_bias) throw RecipeError("selection bias is passed to route(), not bound here");
        Model m = *this;
        Block b;
        b.kind = Block::Moe;
        b.moe = t; b.experts = experts; b.top_k = top_k; b.hidden = hidden; b.ffn = ffn;
        b.scoring = scoring; b.renormalize = renormalize; b.shared = shared; b.scale = scale;
        m.blocks.push_back(b);
        return m;
    }
    Placed place(int device) const;
};

// A model resident on one device (Placed, recipe.rs:21314-21490).
class Placed {
  public:
    Placed(const Model& model, int device) : model_(model) {
        require(rq_init(device, &ctx_));
        try {
            for (const Block& b : model_.blocks) {
                if (b.kind == Block::Layer) {
                    rq_weight* w = nullptr;
                    require(rq_weight_prepare(ctx_, b.tensor.ggml_type, b.tensor.blocks, b.tensor.rows, b.tensor.cols, 0, b.tensor.rows, &w));
                    weights_.push_back(w);
                    banks_.push_back(nullptr);
                    resident_ += (size_t)rq_weight_bytes(w);
                } else {
                    rq_moe* m = nullptr;
                    const bool sh = b.shared.kind == SharedExpert::Gated;
                    require(rq_moe_prepare(ctx_, b.moe.ggml_type, b.moe.gate, b.moe.up, b.moe.down, b.experts, 0, b.experts, b.hidden, b.ffn, sh ? b.moe.shared_gate : nullptr,
                                           sh ? b.moe.shared_up : nullptr, sh ? b.moe.shared_down : nullptr, sh ? b.moe.shared_gate_vector : nullptr, &m));
                    weights_.push_back(nullptr);
                    banks_.push_back(m);
                    resident_ += (size_t)rq_moe_bytes(m);
                }
            }
        } catch (...) {
            release();
            throw;
        }
    }
    Placed(const Placed&) = delete;
    Placed& operator=(const Placed&) = delete;
    ~Placed() { release(); }

    // One position through the chain of layers: input of the first block's width, output of the
    // last block's. Host numbers are f64 (Placed::infer, recipe.rs:21451).
    std::vector<double> infer(const std::vector<double>& input) { return run(input, nullptr); }
    // The same with the router scores of the (single) gguf_moe block of the chain.
    std::vector<double> infer(const std::vector<double>& input, const std::vector<double>& router_scores) { return run(input, &router_scores); }
    void clear() {}                                              // no carried state on this path
    std::vector<size_t> resident_bytes() const { return {resident_}; }
    size_t moved_bytes() const { return moved_; }

  private:
    std::vector<double> run(const std::vector<double>& input, const std::vector<double>* scores) {
        std::vector<float> cur(input.begin(), input.end());
        for (size_t i = 0; i < model_.blocks.size(); ++i) {
            const Block& b = model_.blocks[i];
            if (b.kind == Block::Layer) {
                if ((int64_t)cur.size() != b.tensor.cols) throw RecipeError("input width " + std::to_string(cur.size()) + " does not match the layer's " + std::to_string(b.tensor.cols));
                std::vector<float> out((size_t)b.tensor.rows);
                require(rq_matvec_host(ctx_, weights_[i], cur.data(), 1, b.tensor.cols, 1, out.data(), 1, b.tensor.rows, b.act_mode, b.step));
                moved_ += 4 * (cur.size() + out.size());
                cur.swap(out);
            } else {
                if (!scores || (int)scores->size() != b.experts) throw RecipeError("a gguf_moe block needs one router score per expert");
                if ((int)cur.size() != b.hidden) throw RecipeError("input width does not match the expert bank's hidden width");
                std::vector<float> sc(scores->begin(), scores->end()), out((size_t)b.hidden);
                DeviceBuffer dx(cur.size() * 4), ds(sc.size() * 4), dw(sc.size() * 4), dy(out.size() * 4);
                cuda(cudaMemcpy(dx.p, cur.data(), cur.size() * 4, cudaMemcpyHostToDevice));
                cuda(cudaMemcpy(ds.p, sc.data(), sc.size() * 4, cudaMemcpyHostToDevice));
                require(rq_moe_route(ctx_, (const float*)ds.p, 1, 1, b.experts, b.top_k, (int)b.scoring, b.renormalize ? 1 : 0, nullptr, 1, (float*)dw.p, 1, 1, nullptr));
                require(rq_moe_forward(ctx_, banks_[i], (const float*)dx.p, 1, 1, (const float*)dw.p, 1, 1, b.top_k, 1, 1, (float*)dy.p, 1, 1, nullptr));
                require(rq_check(ctx_));
                cuda(cudaMemcpy(out.data(), dy.p, out.size() * 4, cudaMemcpyDeviceToHost));
                if (b.scale != 1.0) throw RecipeError("a routed scale other than 1 is not served");
                moved_ += 4 * (cur.size() + sc.size() + out.size());
                cur.swap(out);
            }
        }
        return std::vector<double>(cur.begin(), cur.end());
    }
    struct DeviceBuffer {
        void* p = nullptr;
        explicit DeviceBuffer(size_t n) { if (cudaMalloc(&p, n) != cudaSuccess) throw RecipeError("device allocation failed"); }
        ~DeviceBuffer() { cudaFree(p); }
    };
    static void cuda(cudaError_t e) { if (e != cudaSuccess) throw RecipeError(cudaGetErrorString(e)); }
    void release() {
        for (rq_weight* w : weights_) if (w) rq_weight_free(ctx_, w);
        for (rq_moe* m : banks_) if (m) rq_moe_free(ctx_, m);
        weights_.clear(); banks_.clear();
        if (ctx_) rq_destroy(ctx_);
        ctx_ = nullptr;
    }
    Model model_;
    rq_ctx* ctx_ = nullptr;
    std::vector<rq_weight*> weights_;
    std::vector<rq_moe*> banks_;
    size_t resident_ = 0, moved_ = 0;
};

inline Placed Model::place(int device) const { return Placed(*this, device); }  // guaranteed elision: Placed is neither copied nor moved

}  // namespace recipe
