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
