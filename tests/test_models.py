"""Model zoo builders (reference: lib/models/test)."""
import pytest

from flexflow_train_b200 import _ffcore as c


def count(g, t):
    return sum(1 for n in g.nodes() if n["type"] == t)


def test_default_configs_match_reference():
    t = c.default_model_config("transformer")
    assert (t["num_features"], t["sequence_length"], t["batch_size"], t["dim_feedforward"], t["num_heads"]) == (512, 512, 64, 2048, 8)
    assert (t["num_encoder_layers"], t["num_decoder_layers"], t["vocab_size"], t["dropout"]) == (6, 6, 64, 0.1)
    b = c.default_model_config("bert")
    assert (b["vocab_size"], b["hidden_size"], b["num_encoder_layers"], b["num_heads"], b["dim_feedforward"]) == (30522, 768, 12, 12, 3072)
    d = c.default_model_config("dlrm")
    assert d["embedding_size"] == [1000000] * 4 and d["embedding_dim"] == 64 and d["arch_interaction_op"] == "CAT"
    assert c.default_model_config("inception_v3") == {"num_classes": 1000, "batch_size": 32, "aux_logits": True}


def test_transformer_structure():
    g = c.build_model("transformer", None)
    assert count(g, "MULTIHEAD_ATTENTION") == 6 + 12 and count(g, "LAYERNORM") == 12 + 18
    assert count(g, "LINEAR") == 2 * 12 + 1 and count(g, "SOFTMAX") == 1
    out = [n for n in g.nodes() if n["name"] == "out_prob"][0]
    assert out["outputs"][0][1].sizes == [64, 512, 64]


def test_bert_and_lm_variants():
    g = c.build_model("bert", {"batch_size": 2})
    assert count(g, "MULTIHEAD_ATTENTION") == 12 and count(g, "EMBEDDING") == 0
    g = c.build_model("bert", {"batch_size": 2, "token_ids": True, "num_encoder_layers": 2})
    assert count(g, "EMBEDDING") == 2 and count(g, "MULTIHEAD_ATTENTION") == 2
    g = c.build_model("transformer_lm", {"batch_size": 2, "num_decoder_layers": 3})
    assert count(g, "EMBEDDING") == 1 and count(g, "MULTIHEAD_ATTENTION") == 3


def test_inception_v3_shapes():
    g = c.build_model("inception_v3", {"batch_size": 2})
    assert count(g, "CONV2D") == 94 + 2  # 94 in the trunk, 2 in the auxiliary head
    assert count(g, "BATCHNORM") == count(g, "CONV2D")
    out = [n for n in g.nodes() if n["name"] == "out_prob"][0]
    assert out["outputs"][0][1].sizes == [2, 1000]
    flats = [n for n in g.nodes() if n["type"] == "FLAT"]
    assert sorted(n["outputs"][0][1].sizes[1] for n in flats) == [768, 2048]


def test_dlrm_cat_and_dot():
    g = c.build_model("dlrm", {"batch_size": 8, "embedding_size": [1000, 1000]})
    assert count(g, "EMBEDDING") == 2 and count(g, "CONCAT") == 1
    cfg = {"batch_size": 8, "embedding_size": [1000] * 8, "dense_arch_layer_sizes": [13, 512, 256, 64],
           "over_arch_layer_sizes": [0, 512, 256, 1], "arch_interaction_op": "DOT", "final_activation": "SIGMOID",
           "embedding_data_type": "FLOAT"}
    g = c.build_model("dlrm", cfg)
    assert count(g, "BATCHMATMUL") == 1
    last = [n for n in g.nodes() if n["type"] == "LINEAR"][-1]
    assert last["attrs"]["activation"] == "SIGMOID" and last["outputs"][0][1].sizes == [8, 1]


def test_candle_uno_and_split_test():
    g = c.build_model("candle_uno", {"batch_size": 4})
    assert count(g, "INPUT") == 7 and count(g, "CONCAT") == 1
    g = c.build_model("split_test", {"batch_size": 8})
    assert count(g, "LINEAR") == 5 and count(g, "EW_ADD") == 2


def test_unknown_model():
    with pytest.raises(c.CoreError):
        c.build_model("nope", None)
