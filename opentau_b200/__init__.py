"""opentau_b200 — a Blackwell (sm_100a) native framework for training, evaluating and serving
vision-language-action policies (pi0 / pi0.5 / pi0.6 / pi0.7 / cosmos3 / value), with the public
surface of TensorAuto/OpenTau: config schema, batch format, loss dictionary, checkpoint layout."""

__version__ = "0.1.0"

available_policies = ["pi0", "pi05", "pi05_mem", "pi06", "pi07_high_level", "pi07_low_level",
                      "pi07_paligemma_high_level", "pi07_paligemma_low_level", "cosmos3", "cosmos3_nano", "value"]
