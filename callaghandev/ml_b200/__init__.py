"""callaghandev.ml_b200 -- B200 (sm_100a) training back end for CallaghanDev.ML.

``CudaB200AccelerationManager`` mirrors the reference's IAccelerationManager for the training hot path;
``B200LanguageModelTrainer`` / ``B200MlpBatchTrainer`` are the device-resident train-step hooks;
``DataParallelLMTrainer`` (one process per GPU) and ``B200DataParallelGroup`` (one process, all GPUs) shard a batch
over the library's own NCCL data-parallel layer.  Everything runs in libcallaghan_b200.so
(hand-written CUDA); importing this package fails if the library has not been built.
"""
from ._lib import ACT, COST, GEMM_AUTO, GEMM_FP32_SIMT, GEMM_TF32_TCGEN05, B200Error, LMConfig, load
from .manager import CudaB200AccelerationManager
from .trainer import B200DataParallelGroup, B200LanguageModelTrainer, B200MlpBatchTrainer, DataParallelLMTrainer, make_config, split_sequences

load()  # fail loudly at import time when the shared library is missing

__all__ = ["ACT", "COST", "GEMM_AUTO", "GEMM_FP32_SIMT", "GEMM_TF32_TCGEN05", "B200Error", "LMConfig", "load", "CudaB200AccelerationManager",
           "B200DataParallelGroup", "B200LanguageModelTrainer", "B200MlpBatchTrainer", "DataParallelLMTrainer", "make_config", "split_sequences"]
