"""Decoding through the reference's UNCHANGED model runtime (model_hub/LLM.py, model_hub/qwen.py, staged under
baseline/_ref by baseline/stage_reference.py) with this package installed under the reference's module names.

The runtime's files are used as they are.  Two things around them are supplied by the test, because the container has
neither model weights nor the `accelerate` package that `from_pretrained(device_map=...)` needs, and its transformers
release no longer exposes `config.rope_theta`: a tiny random-init Qwen3 checkpoint directory, a loader that builds the
model from that directory's config, and a config loader that puts the `rope_theta` attribute back.  Everything between the
token ids and the logits - embedding, norms, RoPE, projections, `kv_cache.prefill_update_kv_cache /
decode_update_kv_cache`, `polar_prefill_attn / polar_decode_attn`, the MLP - is the reference's own code path.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
DEV = "cuda:0"
ATTN = {"PolarANN": {"core": 0, "nprobe": 0, "cache_unit_size": 0, "cache_cluster_num": 0, "sink_size": 4, "local_size": 16,
                     "dynamic_update_interval": 8, "final_topk": 32, "enable_offload": True}}


@pytest.fixture(scope="module")
def runtime(tmp_path_factory):
    if not os.path.exists(os.path.join(REF, "model_hub", "qwen.py")):
        pytest.skip("the reference's model_hub is not staged under baseline/_ref (python baseline/stage_reference.py)")
    try:
        import flashinfer  # noqa: F401  (the reference's runtime uses it for RMSNorm, RoPE and SiLU)
        from tokenizers import Tokenizer
        from tokenizers.models import WordLevel
        from transformers import AutoConfig, PreTrainedTokenizerFast, Qwen3Config, Qwen3ForCausalLM
    except Exception as e:  # pragma: no cover - depends on the image
        pytest.skip(f"a dependency of the reference's runtime does not import here: {type(e).__name__}: {e}")
    import pariskv_b200.dropin as dropin
    dropin.install(force=True)
    if REF not in sys.path:
        sys.path.insert(0, REF)
    for name in [n for n in sys.modules if n == "model_hub" or n.startswith("model_hub.")]:
        del sys.modules[name]
    import model_hub.qwen as rq
    assert os.path.realpath(rq.__file__).startswith(os.path.realpath(REF))
    d = str(tmp_path_factory.mktemp("ckpt") / "Tiny-Qwen3-1B")     # the runtime parses the model size from "<n>B"
    os.makedirs(d)
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=8192, rope_theta=1.0e6,
                      tie_word_embeddings=False, eos_token_id=1)
    cfg.save_pretrained(d)
    vocab = {f"t{i}": i for i in range(1, 512)}
    vocab["<unk>"] = 0
    PreTrainedTokenizerFast(tokenizer_object=Tokenizer(WordLevel(vocab, unk_token="<unk>")), eos_token="t1",
                            unk_token="<unk>").save_pretrained(d)
    built = {}

    class Loader:   # stands in for AutoModelForCausalLM: random-init weights from the checkpoint's config
        @staticmethod
        def from_pretrained(name, dtype=None, device_map=None, **_):
            torch.manual_seed(1234)
            m = Qwen3ForCausalLM(AutoConfig.from_pretrained(name))
            inv_freq = m.model.rotary_emb.inv_freq.clone()          # from_pretrained keeps this buffer in fp32
            m = m.to(dtype).to(device_map if device_map != "auto" else DEV)
            m.model.rotary_emb.inv_freq = inv_freq.to(m.device)
            m.eval()
            built["hf"] = m
            built["state"] = {k: v.clone() for k, v in m.state_dict().items()}
            return m

    class ConfigLoader:   # stands in for AutoConfig: newer transformers keep rope_theta inside rope_parameters only
        @staticmethod
        def from_pretrained(name, **kw):
            c = AutoConfig.from_pretrained(name, **kw)
            if not hasattr(c, "rope_theta"):
                c.rope_theta = c.rope_parameters["rope_theta"]
            return c

    rq.AutoModelForCausalLM = Loader
    rq.AutoConfig = ConfigLoader
    model = rq.QwenModel(d, 4096, torch.bfloat16, DEV)
    hf = Qwen3ForCausalLM(AutoConfig.from_pretrained(d))           # the runtime strips its copy: a second one to compare with
    inv_freq = hf.model.rotary_emb.inv_freq.clone()
    hf = hf.to(torch.bfloat16).to(DEV).eval()
    hf.model.rotary_emb.inv_freq = inv_freq.to(DEV)
    hf.load_state_dict(built["state"])
    return rq, model, hf


def _dense_logits(hf, ids):
    with torch.no_grad():
        return hf(input_ids=ids, attention_mask=torch.ones_like(ids)).logits[:, -1].float()


def test_short_context_decodes_like_the_dense_model(runtime):
    """300-token prompt (below the full-attention threshold): the cache attends every token, so the logits of the
    prefill and of four decode steps must match the same weights run through a dense causal model, within bf16 noise."""
    rq, model, hf = runtime
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(2, 512, (1, 300), generator=g).to(DEV)
    seen = []
    lm = model.lm
    model.lm = lambda h: seen.append(lm(h)) or seen[-1]
    try:
        out, _ = model.generate("PolarANN", ids, torch.ones_like(ids), max_new_length=5, attn_config=ATTN,
                                disable_early_stop=True)
    finally:
        model.lm = lm
    assert type(model.kv_cache).__module__ == "pariskv_b200.cache_hub.polar_cache"
    assert len(seen) == 5 and len(out[0]) == 5
    cur = ids
    for step, logits in enumerate(seen):
        ref = _dense_logits(hf, cur)
        got = logits.float().view(1, -1)
        tol = 0.05 * ref.abs().max().item() + 0.02
        assert (got - ref).abs().max().item() <= tol, (step, (got - ref).abs().max().item(), tol)
        cur = torch.cat([cur, torch.tensor([[out[0][step]]], device=DEV)], 1)
    assert model.kv_cache.context == 300 + 4


def test_long_context_retrieves_what_the_oracle_retrieves(runtime, oracle):
    """2600-token prompt (above the threshold): every decode step of every layer goes through the retrieval chain.
    The queries that the reference's runtime hands to polar_decode_attn are recorded; for each the cache's selected
    indices must equal the oracle's selection over the keys that the runtime itself put into the cache."""
    rq, model, hf = runtime
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(2, 512, (1, 2600), generator=g).to(DEV)
    calls = []
    real = rq.polar_decode_attn

    def spy(query_states, key_states, value_states, layer_idx, kv_cache):
        res = real(query_states, key_states, value_states, layer_idx, kv_cache)
        calls.append((layer_idx, query_states.detach().cpu().clone(), kv_cache.last_topk_indices.cpu().clone(),
                      kv_cache.zone_len[layer_idx][0]))
        return res

    rq.polar_decode_attn = spy
    try:
        out, _ = model.generate("PolarANN", ids, torch.ones_like(ids), max_new_length=12, attn_config=ATTN,
                                disable_early_stop=True)
    finally:
        rq.polar_decode_attn = real
    cache = model.kv_cache
    assert len(calls) == 11 * 2 and cache.zone_len[0][0] == 2600 - 20 + 8, "eleven decode steps, one flush"
    signs = cache.srht_diagonal_signs.cpu()
    torch.cuda.synchronize()
    for layer_idx, q, final, N in calls:
        zk = cache.unified_keys_cpu[layer_idx][:, :, :N].contiguous()
        cb, w, pk = oracle.encode(zk, signs)
        _, C, Kf = cache.retrieval_plan(N)
        _, coll = cache._get_adaptive_ratios(N)
        r = oracle.retrieve(q.view(1, 1, 8, 128), signs, cb, w, pk, oracle.cluster_counts(cb), cache._mag_centers.cpu(), coll, C, Kf)
        assert torch.equal(final, r["final"]), layer_idx
    cache.check_status()
