"""ctypes signatures of libsp3cuda.so (csrc/kernels)."""

_SDDMM = "i64 p p p p i64 p i64 int p p"
_ROWS = "int i64 p p i64 p i64 int p"
_FILL = "p i64 i64 int i64 i64 int f64 u64 u64 p p"

CUDA_SIGS = {
    "sp3_cuda_sddmm_f32": ("int", _SDDMM),
    "sp3_cuda_sddmm_f64": ("int", _SDDMM),
    "sp3_cuda_spmm_f32": ("int", "int int p p p p p i64 int f32 p i64 p p p p i64 int p p"),
    "sp3_cuda_spmm_f64": ("int", "int int p p p p p i64 int f64 p i64 p p p p i64 int p p"),
    "sp3_cuda_rows_f32": ("int", _ROWS),
    "sp3_cuda_rows_f64": ("int", _ROWS),
    "sp3_cuda_fill_rows_f32": ("int", _FILL),
    "sp3_cuda_fill_rows_f64": ("int", _FILL),
    "sp3_cuda_sum_f32": ("int", "p i64 p p p"),
    "sp3_cuda_sum_f64": ("int", "p i64 p p p"),
    "sp3_cuda_check_range": ("int", "i64 p int int p p"),
    "sp3_cuda_remap": ("int", "i64 p p i64 p p p"),
    "sp3_cuda_invert_perm": ("int", "i64 p p p p"),
    "sp3_cuda_touch_masks": ("int", "i64 p p p p p p p"),
    "sp3_cuda_sddmm_tma_f32": ("int", "i64 p p p p i64 p i64 i64 int p p p"),
    "sp3_cuda_spmm_tma_f32": ("int", "i64 p p p p i64 i64 int f32 p i64 i64 p p"),
    "sp3_cuda_sddmm_orig_f32": ("int", "i64 p p p p i64 p i64 int p p p"),
    "sp3_cuda_sddmm_panel_f32": ("int", "int p p p p p p p p i64 int p i64 int p p p"),
    "sp3_cuda_spmm_panel_f32": ("int", "int p p p p p p p p p i64 int p i64 int p p"),
    "sp3_fused_struct_sizes": ("int", "p p p"),
    "sp3_fused_sddmm_f32": ("int", "p p"),
    "sp3_fused_spmm_f32": ("int", "p p"),
    "sp3_fused_sddmm_f64": ("int", "p p"),
    "sp3_fused_spmm_f64": ("int", "p p"),
    "sp3_fused_ctrl_words": ("int", ""),
    "sp3_symm_alloc": ("int", "u64 p"),
    "sp3_symm_free": ("int", "p"),
    "sp3_ipc_get_handle": ("int", "p p"),
    "sp3_ipc_open": ("int", "p p"),
    "sp3_ipc_close": ("int", "p"),
    "sp3_can_access_peer": ("int", "int int p"),
    "sp3_cuda_error_string": ("s", "int"),
    "sp3_cuda_wait_flag": ("int", "p int u64 p p"),
    "sp3_cuda_signal_flags": ("int", "p int int int p"),
}
