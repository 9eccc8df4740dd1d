"""Random weights are the same bits on the CPU and on the GPU, and -- resting on that -- the engine with all
24 layers of the Qwen1.5-MoE-A2.7B sizes, its weights drawn on the device, against the plain implementation
whose weights are drawn tensor by tensor as it reads them."""
import pytest
import torch

import plain_qwen2moe as plain
from test_engine_gpu import TOL
from tiny_configs import random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("shape,init", [((5,), "bias"), ((64, 130), "linear"), ((3000,), "norm"), ((1100, 1000), "linear")])
def test_random_tensor_cpu_equals_gpu_bit_for_bit(shape, init, monkeypatch):
    from locus_b200.weights import random_init as R

    monkeypatch.setattr(R, "SLICE", 1 << 18)  # several slices in the largest case, cut differently from the default
    for dtype in (torch.float32, torch.bfloat16):
        a = R.random_tensor(4, f"layer.{init}", shape, init, dtype, "cpu")
        b = R.random_tensor(4, f"layer.{init}", shape, init, dtype, DEV)
        assert b.is_cuda and torch.equal(a, b.cpu())
    monkeypatch.undo()
    c = R.random_tensor(4, f"layer.{init}", shape, init, torch.float32, DEV)
    assert torch.equal(c.cpu(), R.random_tensor(4, f"layer.{init}", shape, init, torch.float32, "cpu"))
    # the normal draws themselves, before any rounding, and far into a tensor
    key = R.tensor_key(9, "deep")
    assert torch.equal(R.normal_slice(key, 13_000_000_000, 70000, DEV).cpu(), R.normal_slice(key, 13_000_000_000, 70000, "cpu"))


A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "head_dim": 128, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192, "decoder_sparse_step": 1, "num_experts": 60, "num_experts_per_tok": 4,
    "norm_topk_prob": False, "moe_intermediate_size": 1408, "shared_expert_intermediate_size": 5632,
    "intermediate_size": 5632, "qkv_bias": True, "tie_word_embeddings": False, "use_sliding_window": False,
    "mlp_only_layers": [], "hidden_act": "silu", "eos_token_id": -1,
}
# see tests/test_full_size_gpu.py: what bfloat16 activations do to the router's probabilities
NEAR_TIE = {torch.bfloat16: 3e-2, torch.float32: 1e-5}


class DrawnOnRead:
    """The model's weights as a mapping that draws a tensor on the device when it is read and hands it over
    on the host: nothing of the 14 B parameters is kept."""

    def __init__(self, model, seed, dtype):
        from locus_b200.weights.random_init import random_tensor

        self.src = {s.name: s for _, s in model.tensor_sources()}
        self.draw = lambda s: random_tensor(seed, s.name, s.shape, s.init, dtype, DEV).cpu()

    def __contains__(self, name):
        return name in self.src

    def __getitem__(self, name):
        return self.draw(self.src[name])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_all_24_layers_against_the_plain_implementation(dtype):
    """A 300-token prompt in one step (in bfloat16: tcgen05 attention, grouped expert products on the tensor
    cores; in float32: the CUDA-core path, 57 GB of weights), then two decode steps from the cache, through all
    24 layers; the plain implementation follows the engine's expert choices (checked to be near-ties where they
    differ from its own) and compares logits at sampled positions."""
    import locus_b200.models  # noqa: F401
    from locus_b200.cache import CacheManager
    from locus_b200.config import find_arch
    from locus_b200.engine.step import ModelRunner, StepEntry
    from locus_b200.models.model import Model
    from locus_b200.weights.loader import RandomSource, load_weights

    seed = 2
    entry = find_arch("Qwen2MoeForCausalLM")
    model = Model(entry.build_plan(entry.parse_config(A27B)), dtype, DEV)
    load_weights(model, RandomSource(model, seed, dtype, DEV))
    assert abs(model.param_bytes() / 1e9 - (28.63 if dtype == torch.bfloat16 else 57.26)) < 0.1
    cache = CacheManager(model.cache_needs(), page_tokens=64, n_pages=6, n_state_slots=2, max_seq_tokens=384,
                         dtype=dtype, device=DEV, poison=True)
    runner = ModelRunner(model, cache, max_tokens=320, max_segments=2)
    tokens = random_tokens(302, A27B["vocab_size"], 77)
    places = [0, 1, 63, 64, 127, 200, 299]
    seen = []
    for part in model.all_parts():
        if hasattr(part, "observer"):
            part.observer = lambda prefix, ids, wts: seen.append((prefix, ids.cpu().tolist()))
    seq = cache.open("r")
    got, routed = [], {}
    for a, n, want in ((0, 300, places), (300, 1, [0]), (301, 1, [0])):
        seen.clear()
        assert cache.ensure_capacity(seq, n)
        got.append(runner.step([StepEntry(seq, tokens[a : a + n], want)]).float().cpu().clone())
        for prefix, ids in seen:
            routed.setdefault(prefix, []).extend(ids)
    runner.check_device_errors()
    cache.release(seq)
    got = torch.cat(got).double()
    positions = places + [300, 301]
    del runner, cache
    torch.cuda.empty_cache()

    aux = {}
    ref = plain.forward(A27B, DrawnOnRead(model, seed, dtype), tokens, torch.float64, forced_routing=routed, aux=aux,
                        positions=positions)
    # where the engine chose other experts than the plain router (given the engine's choices before), it was a near-tie
    n_diff = 0
    for prefix, per_pos in aux.items():
        for pos, (ids, probs) in enumerate(per_pos):
            eng = routed[prefix][pos]
            if sorted(eng) != sorted(ids):
                n_diff += 1
                kth = min(float(probs[e]) for e in ids)
                for e in eng:
                    assert float(probs[e]) >= kth * (1 - NEAR_TIE[dtype]), (prefix, pos, e, float(probs[e]), kth)
    # How many may differ: the 4th and 5th best of 60 router logits (sigma 0.9 with these weights) lie about 0.09
    # apart on average, the engine's logits carry an error of sigma 0.007 (bfloat16 activations), so a swap is
    # expected at about 0.8 * 0.007 / 0.09 = 6 % of the (layer, position) pairs; far more would be a fault.
    assert n_diff < (0.10 * 24 * 302 if dtype == torch.bfloat16 else 4), f"{n_diff} choices differ"
    tol_max, tol_mean = TOL[dtype]
    scale = float(ref.abs().max())
    err = (got - ref).abs()
    assert torch.isfinite(got).all()
    assert float(err.max()) <= tol_max * scale, f"max error {float(err.max()):.3e} > {tol_max * scale:.3e}"
    assert float(err.mean()) <= tol_mean * scale, f"mean error {float(err.mean()):.3e}"
