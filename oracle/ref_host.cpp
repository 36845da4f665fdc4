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
// layout operators of the host backend (family_lowering_test_backend.h:77-88, :114-121, :150-154; it has no concat)
int refh_permute(const float* x, int rank, const int64_t* shape, const int64_t* axes, float* out) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.permute(wrap(x, std::vector<int64_t>(shape, shape + rank)), std::vector<int64_t>(axes, axes + rank)), out);
    });
}
int refh_slice(const float* x, int rank, const int64_t* shape, int64_t axis, int64_t start, int64_t stop, float* out) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.slice(wrap(x, std::vector<int64_t>(shape, shape + rank)), axis, start, stop), out);
    });
}
int refh_sinusoidal(const float* positions, int64_t count, int64_t width, int flip, double shift, float* out) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.sinusoidal_embedding(wrap(positions, {count}), width, flip != 0, shift, true), out);
    });
}
// the one padding the host backend implements: constant padding after axis 1 of a [1, rows, width] tensor
int refh_pad_rows(const float* x, int64_t rows, int64_t width, int64_t after, float value, float* out) {
    return guarded([&] {
        family_test::Backend be;
        copy_out(be.pad(wrap(x, {1, rows, width}), {0, 0, 0, after}, value, PadMode::Constant), out);
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


// ---- failure semantics of vrhino_b200::evaluate_fused, exercised on the host --------------------
// The fused chains are stood in for by compositions of the reference's own seams over the test
// backends, so a failure can be injected into any backend call -- inside a fused chain too --
// without a GPU: TinyBackend (native/tests/neural_graph_test_backend.h) throws at its fail_call-th
// primitive, returns broken metadata at its fault_call-th, and fails its synchronize() on request.
namespace {
struct SeamFused final : vrhino_b200::FusedOperators {
    Backend& be;
    std::vector<Tensor> interior;   // the test backends want every tensor they produced alive until the drain
    Tensor hold(Tensor t) { interior.push_back(t); return t; }
    PrecisionPolicy policy = PrecisionPolicy::fp32();
    explicit SeamFused(Backend& b) : be(b) {}
    Backend& backend() override { return be; }
    Tensor layer_norm_modulate(const Tensor& x, const Tensor* w, const Tensor* b, float eps, const Tensor& shift, const Tensor& scale,
                               DType output) override {
        return be.cast(hold(modulate(be, policy, hold(be.layer_norm(x, w, b, eps)), shift, scale)), output);
    }
    Tensor rms_norm_modulate(const Tensor& x, float eps, const Tensor& shift, const Tensor& scale, DType output) override {
        return be.cast(hold(modulate(be, policy, hold(be.rms_norm(x, nullptr, eps, -1, DType::F16)), shift, scale)), output);
    }
    Tensor rms_norm_rope(const Tensor& x, const Tensor* w, float eps, const Tensor* c, const Tensor* s, int heads, DType output) override {
        Tensor n = hold(be.rms_norm(x, w, eps, -1, DType::F16));
        Tensor split = hold(be.reshape(n, {x.dim(0), x.dim(1), heads, x.dim(2) / heads}));
        return be.cast(hold(be.reshape(hold(be.rope_nd(split, *c, *s)), x.shape())), output);
    }
    Tensor gated_residual(const Tensor& residual, const Tensor& branch, const Tensor* gate, DType state) override {
        Tensor update = gate ? hold(be.mul(branch, *gate)) : branch;
        Tensor sum = hold(be.add(residual, update));
        return sum.dtype() == state ? sum : be.cast(sum, state);
    }
};

Tensor filled(const std::vector<int64_t>& shape, float value) {
    Tensor t = Tensor::host(shape, DType::F32);
    for (int64_t i = 0; i < t.numel(); ++i) t.data_as<float>()[i] = value + 0.001f * static_cast<float>(i % 7);
    return t;
}
}  // namespace

// scenario 0: the reference's Wan self-attention graph (F32 contract, dim 64, 2 heads, `tokens` rows) on
//             family_test::Backend, its `n`-th primitive call throwing (n == 0: no failure);
// scenario 1: res + branch * gate (one fused gated residual) on TinyBackend with a failing drain;
// scenario 2: the same, first primitive throwing AND the drain failing;
// scenario 3: the same, the fused result coming back with the wrong shape;
// scenario 4: the same, first primitive throwing something that is not a std::exception.
// report: {threw, code, phase, node, value, primitive, synchronize calls, secondary completion recorded,
//          primitive calls made, outputs returned}; -1 stands for "no location".
int refh_fused_faults(int scenario, int64_t tokens, int n, int64_t* report) {
    namespace ng = neural_graph;
    for (int i = 0; i < 10; ++i) report[i] = 0;
    auto note = [&](const ng::GraphError& e) {
        report[0] = 1; report[1] = static_cast<int64_t>(e.code); report[2] = static_cast<int64_t>(e.phase);
        report[3] = e.node ? static_cast<int64_t>(*e.node) : -1;
        report[4] = e.value ? static_cast<int64_t>(*e.value) : -1;
        report[5] = e.primitive ? static_cast<int64_t>(*e.primitive) : -1;
        report[7] = e.secondary_completion.empty() ? 0 : 1;
        g_error = e.what();
    };
    try {
        if (scenario == 0) {
            wan_family::Config config;
            config.dim = 64; config.heads = 2;
            const ng::Graph graph = wan_internal::self_attention_graph(1, tokens, DType::F32, DType::F32, false, config);
            const ng::Description& d = graph.description();
            std::vector<Tensor> inputs, parameters;
            for (ng::ValueId id : d.inputs) inputs.push_back(filled(d.values[id].shape, 0.05f));
            for (ng::ValueId id : d.parameters) parameters.push_back(filled(d.values[id].shape, 0.01f));
            family_test::Backend be;
            be.fail_call = static_cast<size_t>(n);
            SeamFused fused(be);
            try {
                report[9] = static_cast<int64_t>(vrhino_b200::evaluate_fused(fused, graph, inputs, parameters).size());
            } catch (const ng::GraphError& e) { note(e); }
            report[6] = static_cast<int64_t>(be.syncs);
            report[8] = static_cast<int64_t>(be.calls.size());
            return 0;
        }
        ng::Description d;
        d.schema = ng::schema_v1;
        d.execution_dtype = DType::F32;
        d.values = {{{1, 4, 8}}, {{1, 4, 8}}, {{1, 1, 8}}, {{1, 4, 8}}, {{1, 4, 8}}};
        d.inputs = {0, 1};
        d.parameters = {2};
        d.nodes = {{3, ng::Mul{1, 2}}, {4, ng::Add{0, 3}}};
        d.outputs = {4};
        const ng::Graph graph = ng::admit(d);
        ng::test::TinyBackend be;
        be.fail_sync = scenario == 1 || scenario == 2;
        if (scenario == 2 || scenario == 4) be.fail_call = 1;
        be.throw_nonstandard = scenario == 4;
        if (scenario == 3) { be.fault = ng::test::TinyBackend::Fault::Shape; be.fault_call = 2; }
        SeamFused fused(be);
        try {
            report[9] = static_cast<int64_t>(
                vrhino_b200::evaluate_fused(fused, graph, {filled({1, 4, 8}, 1.f), filled({1, 4, 8}, 2.f)}, {filled({1, 1, 8}, 3.f)}).size());
        } catch (const ng::GraphError& e) { note(e); }
        report[6] = static_cast<int64_t>(be.syncs);
        report[8] = static_cast<int64_t>(be.calls.size());
        return 0;
    } catch (const std::exception& e) { g_error = e.what(); return -1; }
}

}  // extern "C"
