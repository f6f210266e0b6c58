// recipe_rq.hpp -- the host side above the C ABI, in C++ (header only).
//
// The reference's host is Rust; where no Rust toolchain exists this header gives the same
// surface for the quantised matvec path: the names, argument meaning and error behaviour of
// recipe's `Block::fp/int`, `Model::layer`, `Model::gguf_moe`, `Placed::infer/prefill/step/decode/
// clear/resident_bytes/moved_bytes` (recipe.rs:14027-14054, :14671, :14722, :21314-21490). As in
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
    enum Kind { None, Ungated, Gated } kind = None;
    int count = 1;  // how many experts it merges: its feed-forward is count times the routed expert width
    static SharedExpert none() { return {}; }
    static SharedExpert ungated(int count) { return {Ungated, count}; }
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
    enum Kind { Layer, Moe, Embed } kind = Layer;
    Tensor tensor{};
    MoeTensors moe{};
    int experts = 0, top_k = 0, hidden = 0, ffn = 0;
    Scoring scoring = Scoring::Softmax;
    bool renormalize = true;
    SharedExpert shared{};
    double scale = 1.0;
    int act_mode = RQ_ACT_FLOAT, step = 32, int_bits = 0;

    Block fp(uint8_t bits) const {
        if (bits != 32) throw RecipeError("fp bits must be 32 on this path");
        Block b = *this;
        b.act_mode = RQ_ACT_FLOAT;
        return b;
    }
    Block int_(uint8_t bits) const {  // `int` is a keyword in C++
        if (bits != 4 && bits != 8 && bits != 16 && bits != 32) throw RecipeError("int bits must be 4, 8, 16, or 32");
        // int(8): storage Q8_0 (Q4_K kept); int(4): storage Q4_1, int8 activation records against four-bit codes (finish_int_sums,
        // recipe.rs:22345-22369; recipe itself lists no NVIDIA capability for int4, recipe.rs:2658-2681: this library follows its
        // CPU path). int(16) and int(32) widen the activations, which this path does not serve.
        if (bits != 8 && bits != 4) throw RecipeError("int(" + std::to_string(bits) + ") is not served on this path; int(8) and int(4) are");
        if (kind == Moe) throw RecipeError("int sums are only for contractions: expert tables keep their activations (recipe.rs:22340)");
        Block b = *this;
        b.act_mode = RQ_ACT_INT8;
        b.int_bits = bits;
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
    // A lookup of token ids in a stored table ([vocab][hidden] blocks): the first block of a model whose input is a sequence
    // of ids (Model::embed / Primitive::Gather over a bound table, recipe.rs:4632-4651).
    Model embed(const Tensor& table) const {
        if (!blocks.empty()) throw RecipeError("an embedding is the first block of its model");
        Model m = *this;
        Block b;
        b.kind = Block::Embed;
        b.tensor = table;
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
                if (b.kind == Block::Layer || b.kind == Block::Embed) {
                    rq_weight* w = nullptr;
                    require(rq_weight_prepare(ctx_, b.tensor.ggml_type, b.tensor.blocks, b.tensor.rows, b.tensor.cols, 0, b.tensor.rows, &w));
                    const bool kept = b.int_bits == 4 ? rq_int4_keeps(b.tensor.ggml_type) != 0 : rq_int8_keeps(b.tensor.ggml_type) != 0;
                    if (b.kind == Block::Layer && b.act_mode == RQ_ACT_INT8 && !kept) {
                        // finish_int_sums (recipe.rs:22345-22369): `.int(8)` keeps Q8_0 and Q4_K, `.int(4)` keeps Q4_1; any other
                        // bound tensor is re-encoded to the precision's storage (Q8_0, Q4_1) once, at load, and the int dot runs over that
                        rq_weight* q8 = nullptr;
                        const int rc = rq_weight_requantize(ctx_, w, b.int_bits == 4 ? RQ_Q4_1 : RQ_Q8_0, &q8, nullptr);
                        if (rc == RQ_OK) cudaDeviceSynchronize();
                        rq_weight_free(ctx_, w);
                        require(rc);
                        w = q8;
                    }
                    weights_.push_back(w);
                    banks_.push_back(nullptr);
                    resident_ += (size_t)rq_weight_bytes(w);
                } else {
                    rq_moe* m = nullptr;
                    require(rq_moe_prepare(ctx_, b.moe.ggml_type, b.moe.gate, b.moe.up, b.moe.down, b.experts, 0, b.experts, b.hidden, b.ffn, nullptr, nullptr, nullptr,
                                           nullptr, &m));
                    weights_.push_back(nullptr);
                    banks_.push_back(m);
                    if (b.shared.kind != SharedExpert::None) {
                        if (b.shared.count == 0) throw RecipeError("shared expert count must be positive");
                        require(rq_moe_attach_shared(ctx_, m, b.shared.kind == SharedExpert::Gated ? 1 : 0, b.shared.count, b.moe.shared_gate, b.moe.shared_up,
                                                     b.moe.shared_down, b.moe.shared_gate_vector));
                    }
                    require(rq_moe_set_routed_scale(m, (float)b.scale));
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
    // The sequence calls (Placed::prefill / step / decode, recipe.rs:21314-21325, :21468): the model's first block is an
    // embedding, its input a sequence of token ids, its output the last block's values (logits) at the last position.
    // prefill fills exactly the supplied prefix; step extends the completed prefix by one id. No block on this path carries
    // state from one position to the next, so a step runs one position and gives the bits the same position gets in a prefill.
    std::vector<double> prefill(const std::vector<uint32_t>& ids) {
        ids_.clear();
        if (ids.empty()) throw RecipeError("token window is outside the placement capacity");
        std::vector<double> logits = run_ids(ids);
        ids_ = ids;
        return logits;
    }
    std::vector<double> step(uint32_t id) {
        if (ids_.empty()) throw RecipeError("step requires a completed prefill");
        std::vector<double> logits = run_ids({id});
        ids_.push_back(id);
        return logits;
    }
    // Greedy autoregressive decode: the prompt is prefilled, then the id of the largest logit (the lowest index on a tie) is
    // appended and stepped, until a `stop` id, `budget` ids, or the end. Returns the generated ids.
    std::vector<uint32_t> decode(const std::vector<uint32_t>& prompt, const std::vector<uint32_t>& stop, size_t budget) {
        std::vector<uint32_t> out;
        std::vector<double> logits = prefill(prompt);
        while (out.size() < budget) {
            uint32_t best = 0;
            for (size_t i = 1; i < logits.size(); ++i) if (logits[i] > logits[best]) best = (uint32_t)i;
            out.push_back(best);
            bool stopped = false;
            for (uint32_t s : stop) stopped = stopped || s == best;
            if (stopped || out.size() == budget) break;
            logits = step(best);
        }
        return out;
    }
    const std::vector<uint32_t>& ids() const { return ids_; }
    void clear() { ids_.clear(); }                               // forgets the sequence; weights stay resident (recipe.rs:21458)
    std::vector<size_t> resident_bytes() const { return {resident_}; }
    size_t moved_bytes() const { return moved_; }

  private:
    // A window of positions through embedding + layers with the planes on the device; returns the last position's output.
    std::vector<double> run_ids(const std::vector<uint32_t>& ids) {
        if (model_.blocks.empty() || model_.blocks[0].kind != Block::Embed) throw RecipeError("the sequence calls take a model whose first block is an embedding");
        const int tokens = (int)ids.size();
        const Block& e = model_.blocks[0];
        std::vector<int32_t> host_ids(ids.size());
        for (size_t i = 0; i < ids.size(); ++i) {
            if ((int64_t)ids[i] >= e.tensor.rows) throw RecipeError("token id " + std::to_string(ids[i]) + " is outside the table's " + std::to_string(e.tensor.rows) + " rows");
            host_ids[i] = (int32_t)ids[i];
        }
        DeviceBuffer dids(ids.size() * 4);
        cuda(cudaMemcpy(dids.p, host_ids.data(), ids.size() * 4, cudaMemcpyHostToDevice));
        int64_t width = e.tensor.cols;
        std::unique_ptr<DeviceBuffer> cur(new DeviceBuffer((size_t)tokens * width * 4));
        require(rq_gather_rows(ctx_, weights_[0], (const int32_t*)dids.p, tokens, (float*)cur->p, 1, width, nullptr));
        for (size_t i = 1; i < model_.blocks.size(); ++i) {
            const Block& b = model_.blocks[i];
            if (b.kind != Block::Layer) throw RecipeError("the sequence calls serve chains of layers");
            if (width != b.tensor.cols) throw RecipeError("input width " + std::to_string(width) + " does not match the layer's " + std::to_string(b.tensor.cols));
            std::unique_ptr<DeviceBuffer> out(new DeviceBuffer((size_t)tokens * b.tensor.rows * 4));
            // token-major planes; a window goes through the matvec entry point, whose positions get the bits a single step gets
            require(rq_matvec(ctx_, weights_[i], (const float*)cur->p, 1, width, tokens, (float*)out->p, 1, b.tensor.rows, b.act_mode, b.step, nullptr));
            cur.swap(out);
            width = b.tensor.rows;
        }
        require(rq_check(ctx_));
        std::vector<float> last((size_t)width);
        cuda(cudaMemcpy(last.data(), (const float*)cur->p + (size_t)(tokens - 1) * width, last.size() * 4, cudaMemcpyDeviceToHost));
        moved_ += 4 * (ids.size() + last.size());
        return std::vector<double>(last.begin(), last.end());
    }
    std::vector<double> run(const std::vector<double>& input, const std::vector<double>* scores) {
        std::vector<float> cur(input.begin(), input.end());
        for (size_t i = 0; i < model_.blocks.size(); ++i) {
            const Block& b = model_.blocks[i];
            if (b.kind == Block::Embed) throw RecipeError("a model that begins with an embedding takes ids: use prefill / step / decode");
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
    std::vector<uint32_t> ids_;  // the completed prefix (DecodeState.ids, recipe.rs:21316)
};

inline Placed Model::place(int device) const { return Placed(*this, device); }  // guaranteed elision: Placed is neither copied nor moved

}  // namespace recipe
