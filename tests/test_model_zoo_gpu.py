"""Every model family trains on the GPU executor: a few optimizer steps on one fixed batch lower the loss."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from flexflow_train_b200 import _ffcore as core  # noqa: E402
from flexflow_train_b200.ops import kernels as K  # noqa: E402
from flexflow_train_b200.runtime.executor import ExecConfig, Executable, OptimizerConfig  # noqa: E402

CASES = {
    "dlrm_cat": ("dlrm", {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 2, "embedding_size": [1000, 500, 300],
                          "dense_arch_layer_sizes": [13, 64, 16], "over_arch_layer_sizes": [64, 64, 32, 1],
                          "arch_interaction_op": "CAT"}, "mean_squared_error_avg_reduce"),
    "dlrm_dot": ("dlrm", {"batch_size": 64, "embedding_dim": 16, "embedding_bag_size": 1, "embedding_size": [1000, 500, 300],
                          "dense_arch_layer_sizes": [13, 64, 16], "over_arch_layer_sizes": [64, 64, 32, 1],
                          "arch_interaction_op": "DOT"}, "mean_squared_error_avg_reduce"),
    "candle_uno": ("candle_uno", {"batch_size": 32, "dense_layers": [128, 128], "dense_feature_layers": [128, 128],
                                  "feature_shapes": {"dose": 1, "cell.rnaseq": 96, "drug.descriptors": 160, "drug.fingerprints": 64},
                                  "dropout": 0.1}, "mean_squared_error_avg_reduce"),
    "bert": ("bert", {"batch_size": 4, "sequence_length": 64, "hidden_size": 128, "num_heads": 4, "dim_feedforward": 256,
                      "num_encoder_layers": 2, "vocab_size": 512, "token_ids": True, "hidden_dropout_prob": 0.0,
                      "attention_probs_dropout_prob": 0.0, "classifier_dropout": 0.0}, "sparse_categorical_crossentropy"),
    "bert_features": ("bert", {"batch_size": 4, "sequence_length": 64, "hidden_size": 128, "num_heads": 4, "dim_feedforward": 256,
                               "num_encoder_layers": 1, "vocab_size": 512, "hidden_dropout_prob": 0.0,
                               "attention_probs_dropout_prob": 0.0, "classifier_dropout": 0.0}, "sparse_categorical_crossentropy"),
    "transformer": ("transformer", {"num_encoder_layers": 1, "num_decoder_layers": 1, "num_features": 128, "num_heads": 4,
                                    "sequence_length": 32, "batch_size": 4, "dim_feedforward": 256, "vocab_size": 64, "dropout": 0.0},
                    "sparse_categorical_crossentropy"),
    "split_test": ("split_test", {"batch_size": 32}, "sparse_categorical_crossentropy"),
}


def _random_batch(g, ex):
    torch.manual_seed(0)
    inputs = {}
    for n in g.nodes():
        if n["type"] != "INPUT":
            continue
        sh = n["outputs"][0][1]
        sizes = [int(s) for s in sh.sizes]
        name = n["name"] or f"input{n['id']}"
        if sh.dtype in ("INT32", "INT64"):
            cons = [c for c in g.nodes() if any(tuple(v) == (n["id"], "OUTPUT") for _, v in c["inputs"])]
            hi = 16
            for c in cons:
                if c["type"] == "EMBEDDING":
                    hi = int(c["attrs"]["num_entries"])
            inputs[name] = torch.randint(0, hi, sizes, device="cuda", dtype=torch.int32 if sh.dtype == "INT32" else torch.int64)
        else:
            inputs[name] = torch.randn(sizes, device="cuda")
    rows, cols = ex.loss_shape
    if ex.cfg.loss == "sparse_categorical_crossentropy":
        labels = torch.randint(0, cols, (rows,), device="cuda", dtype=torch.int32)
    else:
        labels = torch.rand(rows, cols, device="cuda")
    return inputs, labels


@pytest.mark.parametrize("case", list(CASES))
def test_model_trains(case):
    name, cfg, loss = CASES[case]
    g = core.build_model(name, cfg)
    ex = Executable(g, ExecConfig(compute_dtype="bf16", loss=loss, seed=1, optimizer=OptimizerConfig(kind="adam", lr=2e-3)))
    inputs, labels = _random_batch(g, ex)
    losses = []
    for _ in range(12):
        ex.train_step(inputs, labels)
        losses.append(ex.mean_loss())
    assert all(l == l for l in losses), losses
    assert losses[-1] < losses[0], losses
    assert K.gemm_last_error() == 0
