"""CPU oracle of the fused 4-bit AdamW step: test infrastructure only.

Nothing in the shipped package imports this directory.  ``torch_oracle`` restates the reference's
pure-PyTorch path with the reference's own torch operators; ``c_oracle`` is the same arithmetic in
plain C with every rounding explicit (and OpenMP, for the timed CPU baseline).
"""
