"""The analysis half of the graph fusion pass (vrhino_b200/host/graph_fusion_plan.cpp) on the
reference's own production graphs, on CPU: the Wan and LTX self-attention graphs are built by the
reference's code (compiled into oracle/_ref/libvrhino_ref_host.so) and handed to plan_fusion().

Expected chains: Wan = LayerNorm-modulate + RMSNorm-RoPE for q and k + gated residual; LTX =
RMSNorm-modulate + RMSNorm-RoPE for q and k + gated residual.  Under the F32 contract the Wan graph
has no operand cast after RoPE, so its q/k chains stay unfused there; a diagnostics graph exports the
interior values, which must switch the fusion of those chains off."""
import pytest

from oracle import ref


@pytest.fixture(scope="module")
def host():
    if not ref.available_host():
        pytest.skip("oracle/_ref/libvrhino_ref_host.so has not been built (make -C oracle ref_host)")
    h = ref.RefHost()
    if not hasattr(h.lib, "refh_fusion_plan"):
        pytest.skip("host library predates the fusion plan entry")
    return h


@pytest.mark.parametrize("contract,rope_chains", [("f32", 0), ("bf16_f32_hidden", 2), ("bf16", 2)])
def test_wan_production_graph(host, contract, rope_chains):
    plan = host.fusion_plan("wan", contract)
    assert (plan["layer_norm_modulate"], plan["rms_norm_modulate"], plan["rms_norm_rope"], plan["gated_residual"]) == (1, 0, rope_chains, 1)
    assert plan["nodes_absorbed"] >= 4 + 4 * rope_chains
    diag = host.fusion_plan("wan", contract, diagnostics=True)
    assert diag["nodes_absorbed"] == 0 and diag["layer_norm_modulate"] == 0 and diag["rms_norm_rope"] == 0


@pytest.mark.parametrize("contract", ["f32", "bf16_f32_hidden", "bf16"])
def test_ltx_production_graph(host, contract):
    plan = host.fusion_plan("ltx", contract)
    assert (plan["layer_norm_modulate"], plan["rms_norm_modulate"], plan["rms_norm_rope"], plan["gated_residual"]) == (0, 1, 2, 1)
    assert plan["nodes_absorbed"] >= 6
    diag = host.fusion_plan("ltx", contract, diagnostics=True)
    # the diagnostics graph exports the norm, the modulated input and the positioned q / k
    assert diag["rms_norm_modulate"] == 0 and diag["rms_norm_rope"] == 0


def test_evaluate_fused_reports_failures_like_the_reference_evaluator(host):
    """neural_graph::evaluate reports every failure as a GraphError with code, phase and the node /
    value / primitive at work, and drains the device once if work may be in flight
    (native/src/runtime/neural_graph_evaluator.cpp:84-93, :162-175).  evaluate_fused does the same;
    the failures are injected on the host through the reference's own test backends."""
    clean = host.fused_faults(0, tokens=4, n=0)
    assert not clean["threw"] and clean["outputs"] == 2 and clean["syncs"] == 1
    calls = clean["calls"]
    assert calls > 10
    seen_nodes = set()
    for n in range(1, calls + 1):                       # a failure in every single backend call of the graph
        r = host.fused_faults(0, tokens=4, n=n)
        assert r["threw"] and r["code"] == "BackendFailure" and r["phase"] == "Run", (n, r)
        assert r["node"] is not None and r["value"] is not None and r["primitive"] is not None, (n, r)
        assert r["syncs"] == 1, (n, r)                   # drained exactly once after the failure
        assert "injected primitive failure" in r["text"]
        seen_nodes.add(r["node"])
    assert len(seen_nodes) >= 8                          # failures were attributed to many different nodes
    r = host.fused_faults(1)                             # the drain itself fails
    assert r["threw"] and r["code"] == "CompletionFailure" and r["phase"] == "Drain" and r["node"] is None and r["syncs"] == 1
    r = host.fused_faults(2)                             # a primitive fails, then the drain after it fails too
    assert r["code"] == "BackendFailure" and r["phase"] == "Run" and r["secondary_completion"] and r["syncs"] == 1
    assert r["node"] == 1                                # the fused chain runs at its last node (the Add)
    r = host.fused_faults(3)                             # the fused result has the wrong shape
    assert r["code"] == "InvalidNodeOutput" and r["phase"] == "Run" and r["node"] == 1 and r["syncs"] == 1
    r = host.fused_faults(4)                             # something that is not a std::exception
    assert r["code"] == "BackendFailure" and "Non-standard" in r["text"] and r["syncs"] == 1
