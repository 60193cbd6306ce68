"""Model factory: deterministic initialisation (every node starts from the same weights)."""


def test_two_builds_from_the_same_hparams_are_identical_to_the_last_bit():
    from types import SimpleNamespace

    from templar_b200 import model_factory as mf

    hp = SimpleNamespace(model_size="tiny", sequence_length=32,
                         model_config=SimpleNamespace(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                                                      num_key_value_heads=2, intermediate_size=256, rms_norm_eps=1e-5,
                                                      rope_theta=10000.0), torchtitan=SimpleNamespace())
    rep = mf.check_init(hp)
    assert rep["identical"] and rep["differing"] == [] and len(set(rep["fingerprints"])) == 1
    m = mf.initialize_torchtitan_model(hp, device="cpu")
    assert mf.model_fingerprint(m) == rep["fingerprints"][0]
    import torch

    with torch.no_grad():
        next(m.parameters()).add_(1e-3)
    assert mf.model_fingerprint(m) != rep["fingerprints"][0]
