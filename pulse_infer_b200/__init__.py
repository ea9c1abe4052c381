"""pulse_infer_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

Layout: ``config`` (typed configuration, architecture registry), ``weights`` (safetensors by name,
seeded random weights), ``parts`` (mixer, feed-forward, norm, position encoding, block, and the generic
decoder that runs them), ``models`` (architectures as data), ``cache`` (paged keys/values, block tables,
state slots), ``engine`` (step function, scheduler, replay), ``sampling``, ``ops`` + ``csrc`` (the CUDA
kernels and their Python entry points).
"""
__version__ = "0.1.0"


def __getattr__(name):
    # lazy: importing the package must not need torch.cuda or nvcc
    if name == "Engine":
        from .api import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    raise AttributeError(name)
