"""Model configuration contracts that need no device."""
import pytest


def test_gpt_oss_config_contract(tmp_path):
    import json
    from dataclasses import replace
    from oa_b200.models.gpt_oss import OaGptOssConfig
    c20, c120 = OaGptOssConfig.Preset20B(), OaGptOssConfig.Preset120B()
    assert c20.Validate() == (True, "") and c20.IsPublished20B() and not c20.IsPublished120B() and c120.IsPublished120B()
    assert (c20.QueryWidth(), c20.KvWidth(), c20.ExpectedLogicalWeightCount()) == (4096, 512, 3 + 24 * 19)
    assert c20.LayerUsesSlidingAttention(0) and not c20.LayerUsesSlidingAttention(1)
    assert 20.5e9 < c20.ParameterCount() < 21.5e9 and 115e9 < c120.ParameterCount() < 119e9
    for bad, word in ((replace(c20, NumKvHeads=7), "GQA"), (replace(c20, HeadDim=63), "RoPE"), (replace(c20, ExpertsPerToken=64), "inconsistent"),
                      (replace(c20, EosToken=10 ** 6), "special token"), (replace(c20, TieWordEmbeddings=True), "contract"),
                      (replace(c20, RopeNtkBeta=0.5), "RoPE")):
        ok, msg = bad.Validate()
        assert not ok and word in msg
    small = replace(c20, NumLayers=2, HiddenSize=64, IntermediateSize=64, NumAttentionHeads=8, NumKvHeads=2, HeadDim=16, NumExperts=4,
                    ExpertsPerToken=2, VocabSize=300, PadToken=1, EosToken=2)
    assert small.Validate()[0] and not small.IsPublished20B()
    inv, scale = c20.YarnInverseFrequencies()
    assert len(inv) == 32 and abs(inv[0] - 1.0) < 1e-12 and abs(inv[-1] - 150000.0 ** (-62 / 64) / 32) < 1e-12      # ends: kept / fully interpolated
    assert all(a >= b for a, b in zip(inv, inv[1:])) and abs(scale - (0.1 * 3.4657359 + 1)) < 1e-6
    doc = {"model_type": "gpt_oss", "vocab_size": 201088, "num_hidden_layers": 24, "hidden_size": 2880, "intermediate_size": 2880,
           "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 64, "num_local_experts": 32, "num_experts_per_tok": 4,
           "sliding_window": 128, "initial_context_length": 4096, "max_position_embeddings": 131072, "rope_theta": 150000, "rms_norm_eps": 1e-5,
           "swiglu_limit": 7.0, "pad_token_id": 199999, "eos_token_id": 200002, "attention_bias": True, "tie_word_embeddings": False,
           "rope_scaling": {"factor": 32.0, "beta_slow": 1.0, "beta_fast": 32.0},
           "layer_types": ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(24)],
           "quantization_config": {"quant_method": "mxfp4"}}
    p = tmp_path / "config.json"
    p.write_text(json.dumps(doc))
    assert OaGptOssConfig.FromJson(str(p)).IsPublished20B()
    for key, val, word in (("model_type", "llama", "model_type"), ("layer_types", ["full_attention"] * 24, "alternate"),
                           ("quantization_config", {"quant_method": "fp8"}, "MXFP4"), ("num_key_value_heads", 7, "GQA")):
        p.write_text(json.dumps({**doc, key: val}))
        with pytest.raises(ValueError, match=word):
            OaGptOssConfig.FromJson(str(p))
