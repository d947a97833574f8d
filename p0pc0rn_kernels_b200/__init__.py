"""p0pc0rn-kernels `gemm` for B200: hand-written sm_100a CUDA kernels behind the reference's ``op(gpu, args)`` API.

The names exported here are the reference's (src/index.js) for the gemm path and the model I/O either side of it.
The native library must be built (``python p0pc0rn_kernels_b200/build.py``); there is no CPU fallback."""
from .attention import attention
from .convert import ALIGN, convert, convertSafetensors, encodedBytes, writeSafetensors
from .encode import (MANIFEST_FORMAT, chooseEncoding, dtypeBytes, encodeRows, matrixOf, packF16, packF32, packQ4, packQ8, reorderConvRows,
                     safetensorsHeader, safetensorsList, tileBytes, toFloat32)
from .gemm import DEFAULT_TILE, gemm
from .gpu import MB, Buffer, Gpu, GpuError, createGpu, f2h, fromF16, h2f, toF16, view
from .misc import gnFinalize, gnPartBytes, gnPartial, groupnormStats, pixstats, rowstats
from .shard import (all_gather_columns, all_gather_frames, conv3_frame_shard, shard_bytes, shard_frames, shard_rows, shard_swiglu_bytes,
                    shard_weight)
from .tune import TUNE_TABLE, calibrate, defaultTune, tuneEntry
from .weights import loadWeights, uploadWeights

__all__ = [n for n in dir() if not n.startswith("_")]
