"""atlas_b200 — B200 (sm_100a) implementation of ATLAS's single-token decode path behind the
reference's own tensor / quant / model surface.  See include/atlas_kernels.h for the C ABI."""
from ._ffi import AUTO, AtlasError, BF16, F16, F32, INT4, INT8, cuda_available, cuda_device_count  # noqa: F401
from .tensor import (Context, GpuKvCache, GpuMatrix, GpuRopeTables, GpuVec, device_sync, gpu_argmax,  # noqa: F401
                     qk_norm_inplace_gpu, rope_tables, silu_mul_gpu)
from .quant import INT4_BLOCK_SIZE, Int4Tensor, Int8Tensor  # noqa: F401
from .model import LAYER_FULL, LAYER_SLIDING, ModelConfig, OlmoModel, SamplingConfig, Yarn, sample_token  # noqa: F401
from .infer import InferEngine, PheromoneDeposit, StigmergicHook  # noqa: F401
from .safetensors import (LoadStats, SafetensorsFile, TensorDesc, load_model_from_dir, load_model_from_safetensors,  # noqa: F401
                          patch_config_from_hf_json)
