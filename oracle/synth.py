"""Same seeded generators as the product uses, re-exported for the checker side."""
from gradcraft_b200.synth import *  # noqa: F401,F403
from gradcraft_b200.synth import gpt_param_shapes, gpt_weights, name_seed, normal, token_batches, uniform53, zipf_cdf, zipf_tokens  # noqa: F401
