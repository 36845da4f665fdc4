// C wrapper around the REFERENCE's own host path, compiled from the reference's sources where
// they lie (see oracle/Makefile).  TEST / BASELINE INFRASTRUCTURE ONLY.  The host path is
// family_test::Backend, the F32 single-threaded "synthetic-host" backend of
// native/tests/family_lowering_test_backend.h:11-156, driven through the reference's helper
// seams (native/include/vrhino/architecture.h:63-86) and SamplingPrimitives
// (native/include/vrhino/sampling.h:171-203).  This file contains no reference code.
//
// Rows are independent, so the Wan block chain can be spread over host threads: every thread
// owns its own Backend instance and a contiguous range of token rows.
#include <chrono>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "family_lowering_test_backend.h"
#include "architectures/ltx_self_attention_graph.h"
#include "architectures/wan_self_attention_graph.h"
#include "graph_fusion.h"
#include "vrhino/architecture.h"
#include "vrhino/precision.h"
#include "vrhino/sampling.h"
#include "vrhino/tensor_util.h"

using namespace vrhino;

namespace {
std::string g_error;

Tensor wrap(const float* data, std::vector<int64_t> shape) {
    // borrowed: the reference helpers never write to their inputs
    const size_t bytes = static_cast<size_t>(shape_numel(shape)) * sizeof(float);
    return Tensor::borrowed(const_cast<float*>(data), bytes, std::move(shape), DType::F32);
}
void copy_out(const Tensor& t, float* out) { std::memcpy(out, t.data(), t.bytes()); }

template <typename F>
int guarded(F&& f) {
    try { f(); return 0; } catch (const std::exception& e) { g_error = e.what(); return -1; }
}
}  // namespace

extern "C" {

const char* refh_last_error() { return g_error.c_str(); }

int refh_layer_norm(const float* x, const float* w, const float* b, float* out, int64_t rows, int64_t width, float eps) {
    return guarded([&] {
        family_test::Backend be;
        Tensor wt, bt;
        if (w) wt = wrap(w, {width});
        if (b) bt = wrap(b, {width});
        copy_out(be.layer_norm(wrap(x, {rows, width}), w ? &wt : nullptr, b ? &bt : nullptr, eps), out);
    });
}
int refh_rms_norm(const float* x, const float* w, float* out, int64_t rows, int64_t width, float eps) {
    return guarded([&] {
        family_test::Backend be;
        Tensor wt;
        if (w) wt = wrap(w, {width});
        copy_out(be.rms_norm(wrap(x, {rows, width}), w ? &wt : nullptr, eps, -1, DType::F32), out);
    });
}
int refh_activation(const float* x, float* out, int64_t count, int kind) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.activation(wrap(x, {count}), static_cast<Activation>(kind)), out);
    });
}
// x [1, tokens, heads, width]; cos / sin [1, tokens, 1, width]
int refh_rope(const float* x, const float* c, const float* s, float* out, int64_t tokens, int64_t heads, int64_t width) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.rope_nd(wrap(x, {1, tokens, heads, width}), wrap(c, {1, tokens, 1, width}), wrap(s, {1, tokens, 1, width})), out);
    });
}
int refh_modulate(const float* x, const float* shift, const float* scale, float* out, int64_t rows, int64_t width) {
    return guarded([&] {
        family_test::Backend be;
        const PrecisionPolicy policy = PrecisionPolicy::fp32();
        copy_out(modulate(be, policy, wrap(x, {1, rows, width}), wrap(shift, {1, 1, width}), wrap(scale, {1, 1, width})), out);
    });
}
// gate == nullptr: residual_add
int refh_gated_residual(const float* res, const float* branch, const float* gate, float* out, int64_t rows, int64_t width) {
    return guarded([&] {
        family_test::Backend be;
        const PrecisionPolicy policy = PrecisionPolicy::fp32();
        Tensor r = wrap(res, {1, rows, width}), b = wrap(branch, {1, rows, width});
        copy_out(gate ? gated_residual(be, policy, r, b, wrap(gate, {1, 1, width})) : residual_add(be, policy, r, b), out);
    });
}
int refh_cfg_euler(const float* x, const float* u, const float* c, float* guided, float* out, int64_t count,
                   float scale, float delta) {
    return guarded([&] {
        family_test::Backend be;
        SamplingPrimitives p(be, PrecisionPolicy::fp32());
        Tensor g = p.cfg_combine(wrap(u, {count}), wrap(c, {count}), scale);
        if (guided) copy_out(g, guided);
        copy_out(p.euler_update(wrap(x, {count}), g, scalar_f32(delta), true), out);
    });
}

// The Wan DiT-block non-GEMM chain (native/src/architectures/wan.cpp:68-119 and
// wan_self_attention_graph.h:46-70) on F32 host tensors, `tokens` rows, split over `threads`.
// Inputs: x q k proj cross_q cross ffn_out [tokens, dim]; ffn_hidden [tokens, ffn];
// cross_k [text, dim]; mod [6, dim]; wq wk wcq wck gamma beta [dim]; cos sin [tokens, dim/heads].
// Outputs are discarded (this entry point exists to time the reference's host path); returns
// seconds per step, or a negative value on error.
double refh_wan_chain_seconds(const float* x, const float* q, const float* k, const float* proj, const float* cross_q,
                              const float* cross_k, const float* cross, const float* ffn_out, const float* ffn_hidden,
                              const float* mod, const float* wq, const float* wk, const float* wcq, const float* wck,
                              const float* gamma, const float* beta, const float* cosine, const float* sine,
                              int64_t tokens, int64_t text, int64_t dim, int64_t heads, int64_t ffn,
                              int threads, int steps) {
    if (threads < 1) threads = 1;
    const int64_t d = dim / heads;
    bool failed = false;
    auto work = [&](int t) {
        try {
            family_test::Backend be;
            const PrecisionPolicy policy = PrecisionPolicy::fp32();
            const int64_t r0 = tokens * t / threads, r1 = tokens * (t + 1) / threads, n = r1 - r0;
            const int64_t k0 = text * t / threads, k1 = text * (t + 1) / threads;
            if (n <= 0) return;
            auto rowsof = [&](const float* p, int64_t width) { return wrap(p + r0 * width, {1, n, width}); };
            std::vector<Tensor> m;
            for (int i = 0; i < 6; ++i) m.push_back(wrap(mod + i * dim, {1, 1, dim}));
            Tensor tx = rowsof(x, dim), wqt = wrap(wq, {dim}), wkt = wrap(wk, {dim}), wcqt = wrap(wcq, {dim}), wckt = wrap(wck, {dim});
            Tensor g3 = wrap(gamma, {dim}), b3 = wrap(beta, {dim});
            Tensor co = wrap(cosine + r0 * d, {1, n, 1, d}), si = wrap(sine + r0 * d, {1, n, 1, d});
            auto qk = [&](const float* src, const Tensor& w) {
                Tensor nrm = attention_norm(be, policy, rowsof(src, dim), &w, 1e-6f);
                return operation_rope(be, policy, be.reshape(nrm, {1, n, heads, d}), co, si);
            };
            (void)modulate(be, policy, be.layer_norm(tx, nullptr, nullptr, 1e-6f), m[0], m[1]);          // A
            (void)qk(q, wqt); (void)qk(k, wkt);                                                            // B
            (void)gated_residual(be, policy, tx, rowsof(proj, dim), m[2]);                                 // C
            (void)be.layer_norm(tx, &g3, &b3, 1e-6f);                                                      // D
            (void)attention_norm(be, policy, rowsof(cross_q, dim), &wcqt, 1e-6f);                          // E
            if (k1 > k0) (void)attention_norm(be, policy, wrap(cross_k + k0 * dim, {1, k1 - k0, dim}), &wckt, 1e-6f);
            (void)residual_add(be, policy, tx, rowsof(cross, dim));                                        // F
            (void)modulate(be, policy, be.layer_norm(tx, nullptr, nullptr, 1e-6f), m[3], m[4]);          // G
            (void)be.activation(rowsof(ffn_hidden, ffn), Activation::GeluTanh);                            // H
            (void)gated_residual(be, policy, tx, rowsof(ffn_out, dim), m[5]);                              // I
        } catch (const std::exception& e) { g_error = e.what(); failed = true; }
    };
    const auto t0 = std::chrono::steady_clock::now();
    for (int s = 0; s < steps; ++s) {
        std::vector<std::thread> pool;
        for (int t = 1; t < threads; ++t) pool.emplace_back(work, t);
        work(0);
        for (auto& th : pool) th.join();
    }
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return failed ? -1.0 : seconds / (steps > 0 ? steps : 1);
}


// ---- graph fusion plan on the reference's production graphs (analysis only, no device) ------
// which: 0 Wan self-attention graph (wan_self_attention_graph.h), 1 LTX (ltx_self_attention_graph.cpp).
// contract: 0 F32, 1 BF16 execution with F32 hidden state, 2 BF16 execution with BF16 hidden state.
// out: {layer_norm_modulate, rms_norm_modulate, rms_norm_rope, gated_residual, nodes_total, nodes_absorbed}.
int refh_fusion_plan(int which, int contract, int diagnostics, int64_t tokens, int* out) {
    try {
        const DType execution = contract == 0 ? DType::F32 : DType::BF16;
        const DType hidden = contract == 2 ? DType::BF16 : DType::F32;
        vrhino_b200::FusionPlan plan;
        if (which == 0) {
            plan = vrhino_b200::plan_fusion(wan_internal::self_attention_graph(1, tokens, execution, hidden, diagnostics != 0).description());
        } else {
            const auto c = contract == 0 ? ltx_internal::SelfAttentionContract::F32
                         : contract == 1 ? ltx_internal::SelfAttentionContract::BF16F32Hidden
                                         : ltx_internal::SelfAttentionContract::BF16Hidden;
            plan = vrhino_b200::plan_fusion(ltx_internal::self_attention_graph(2, tokens, 1, diagnostics != 0, false, c).description());
        }
        out[0] = plan.stats.layer_norm_modulate; out[1] = plan.stats.rms_norm_modulate; out[2] = plan.stats.rms_norm_rope;
        out[3] = plan.stats.gated_residual; out[4] = plan.stats.nodes_total; out[5] = plan.stats.nodes_absorbed;
        return 0;
    } catch (const std::exception& e) { g_error = e.what(); return -1; }
}

}  // extern "C"
