"""B200-native sparse-weight x dense-activation SpMM (tiled-CSL, tcgen05), drop-in for the reference's libSpMM_API."""
from .spmm_api import (  # noqa: F401
    LIB_PATH,
    SUPPORTED_N,
    TILE_K,
    TILE_M,
    GenSparseMatrixBinFile,
    InitSparseMatrixA_API,
    InitSparseMatrixA_API_NoReorder,
    SpMM_SplitK_API,
    SpMM_SplitK_API_token_major,
    decompose,
    device_status,
    plan,
    selftest_wait_timeout,
    spmm_own_scratch,
    synth_fp16,
    workspace_bytes,
)
