"""The engine at the layer sizes of real models (one or two layers of each, the full vocabulary), against the plain
implementation run in float64 on the GPU: head size 128, query width unequal to the hidden size, a vocabulary that is no
power of two, tied and untied heads. float32 must agree to 1e-4 relative and give the same greedy tokens for every way
of cutting the work; bfloat16 stays within the bounds stated in tests/helpers.py."""
import pytest
import torch

from roost_b200.engine.executor import StepEntry, StepExecutor
from roost_b200.weights.random_init import write_random_model
from tests import helpers as H
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", rope_theta=1000000.0, rms_norm_eps=1e-6,
            vocab_size=151936, max_position_embeddings=40960, torch_dtype="bfloat16", head_dim=128, num_key_value_heads=8)
SHAPES = {
    "0.6b": dict(BASE, num_hidden_layers=2, hidden_size=1024, num_attention_heads=16, intermediate_size=3072, tie_word_embeddings=True),
    "8b": dict(BASE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(BASE, num_hidden_layers=1, hidden_size=5120, num_attention_heads=64, intermediate_size=25600, tie_word_embeddings=False),
}


@pytest.fixture(scope="module", params=list(SHAPES))
def big(request, tmp_path_factory):
    name = request.param
    d = tmp_path_factory.mktemp(f"big_{name}")
    write_random_model(d, SHAPES[name], seed=11, std=0.02, norm_std=0.05)
    cfg, w = plain.load_model_dir(d)
    w = {k: v.cuda() for k, v in w.items()}       # the plain implementation, in float64, on the GPU
    ids = H.random_ids(80, 151936, seed=12)
    want = plain.forward_logits(cfg, w, ids).cpu()
    del w
    torch.cuda.empty_cache()
    return name, d, ids, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_sizes_of_real_models(big, dtype):
    name, model_dir, ids, want = big
    model = H.make_model(model_dir, dtype, "gpu")
    ex = StepExecutor(model, page_size=16, num_pages=24, max_requests=4)
    whole = H.run_whole(ex, "w", ids).cpu()
    tail = H.run_tail_decoded(ex, "t", ids, tail=32).cpu()
    parts = H.run_portions(ex, "p", ids, [17, 2, 9, 3, 2, 31]).cpu()
    a, b = H.random_ids(40, 151936, 13), H.random_ids(25, 151936, 14)
    mixed = H.run_mixed(ex, {"m": ids, "a": a, "b": b}, seed=15, max_live=3, decode_tail=6)["m"].cpu()
    for what, got in (("whole", whole), ("tail decoded", tail), ("portions", parts), ("mixed", mixed)):
        err, rms = H.scaled_error(got, want), H.rms_error(got, want)
        print(f"MEASURED {name} {dtype} {what}: worst scaled error {err:.3e}, rms error {rms:.3e}")
        if dtype == torch.float32:
            assert err < 1e-4, f"{name} {what}: {err}"
            top2 = want.topk(2, dim=-1).values
            clear = (top2[:, 0] - top2[:, 1]) > 1e-3
            assert torch.equal(got.argmax(-1)[clear], want.argmax(-1)[clear])
        else:
            # twelve million logits are compared here, three hundred times more than on the tiny models: the worst of
            # that many roundings of the same size lies near six standard deviations instead of four (measured 2.9e-2 to
            # 6.8e-2 with a root-mean-square error of 0.9e-2 to 1.1e-2), so the worst-case bound is 2^-3 here; the
            # root-mean-square bound, which does not grow with the sample, stays 2^-6
            assert err < 2.0 ** -3 and rms < H.BF16_RMS_BOUND, f"{name} {what}: worst {err}, rms {rms}"
    if dtype == torch.float32:
        assert torch.equal(tail, whole) and torch.equal(parts, whole) and torch.equal(mixed, whole), \
            "the float32 kernels promise the same bits for every cut"
    assert all(p.free_count == p.capacity for p in ex.cache.pools)
