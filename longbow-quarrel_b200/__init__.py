"""longbow-quarrel_b200: a small, whole model library for the Llama 3 dense decoder
on one B200 -- configuration, weights, layers from parts, a paged cache with a slot
per sequence, one step function, generation and sampling, trace replay -- on
hand-written sm_100a kernels."""
__version__ = "0.1.0"
