"""A single-GPU inference engine for the Qwen3 dense decoder on NVIDIA B200 (sm_100a).

Subpackages, in the order a request meets them:

``config``         typed model and engine configuration, the architecture registry
``weights``        safetensors loading by tensor name, seeded random model folders
``architectures``  one module per architecture: config.json keys -> parts, order, tensor names
``parts``          norm, position encoding, mixer, feed-forward, block; the model assembled from them
``cache``          paged key/value pools per layer group, block tables, state slots, prefix reuse
``engine``         the step function, scheduler, request state, ``LLM`` entry point
``sampling``       sampling parameters and the device sampler
``kernels``        ctypes bindings of the CUDA library built from ``csrc/``
"""

__version__ = "0.1.0"
