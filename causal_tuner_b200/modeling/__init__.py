"""Parameter containers of the hot path: same names as the reference's ``causal_tuner.modeling``."""
