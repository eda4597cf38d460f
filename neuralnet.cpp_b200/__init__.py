"""nn-b200: host-side mirror of the reference's engine / layer operator surface on top of
libnn-b200.so (hand-written CUDA for sm_100a).

The directory name carries a dot, so the package is imported under the module name
``neuralnet_cpp_b200`` (see ``__graft_entry__.load_package``).  Importing it never builds
anything; the shared library must exist (``python neuralnet.cpp_b200/build.py``) and is loaded on
first use.  There is no CPU fallback: without the library, or without a B200, calls raise.
"""
from ._lib import lib, lib_path, NnbError  # noqa: F401
from .engine import Engine  # noqa: F401
from .policy import GptConfig, Policy, SamplingConfig, GELU, SWIGLU, RELU2, LEARNED, ROPE  # noqa: F401
from .grpo import GrpoConfig, GrpoTrainer, hash_reward, report_dict, REPORT_FIELDS  # noqa: F401
from .ppo import PpoConfig, PpoTrainer  # noqa: F401
from .pipeline import (CollectingMetricSink, DeterministicRng, ExperienceBuffer, GptRolloutSource, PipelineError,  # noqa: F401
                       RLPipelineConfig, RLTrainingPipeline, RolloutSource, RolloutSpec, TensorRecord, UniformBatchSampler)
