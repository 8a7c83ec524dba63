"""ctypes signatures of the CUDA library's C API (``csrc/include/rbv/rbruckv.h``)."""
import ctypes as C

c_int_p = C.POINTER(C.c_int)
c_ll_p = C.POINTER(C.c_longlong)


class Status(C.Structure):
    _fields_ = [("code", C.c_int), ("site", C.c_int), ("detail0", C.c_int), ("detail1", C.c_int),
                ("trace", C.c_ulonglong * 8)]


class Box(C.Structure):
    _fields_ = [("n0", C.c_int), ("n1", C.c_int), ("n2", C.c_int), ("src_off", C.c_longlong), ("s0", C.c_longlong),
                ("s1", C.c_longlong), ("dst_off", C.c_longlong), ("t0", C.c_longlong), ("t1", C.c_longlong),
                ("t2", C.c_longlong)]


STATUS_NAMES = {0: "ok", 1: "timeout", 2: "bad_argument", 3: "staging_capacity", 4: "truncate", 5: "aborted"}
SITE_NAMES = {0: "-", 1: "metadata", 2: "staging_cell", 3: "final_arrival", 4: "bulk_copy"}


def declare_cuda(lib):
    lib.rbv_last_error.restype = C.c_char_p
    lib.rbv_ctx_create.restype = C.c_void_p
    lib.rbv_ctx_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_size_t]
    lib.rbv_ctx_destroy.argtypes = [C.c_void_p]
    lib.rbv_ctx_ipc_handle.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_connect.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_set_stream.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_set_timeout_ms.argtypes = [C.c_void_p, C.c_double]
    lib.rbv_ctx_set_launch.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
    lib.rbv_ctx_sync.argtypes = [C.c_void_p]
    lib.rbv_ctx_set_absent_rank.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_ctx_status.argtypes = [C.c_void_p, C.POINTER(Status)]
    lib.rbv_ctx_reset.argtypes = [C.c_void_p]
    lib.rbv_ctx_info.argtypes = [C.c_void_p, c_ll_p]
    lib.rbv_ctx_heap.restype = C.c_void_p
    lib.rbv_ctx_heap.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_symm_alloc.restype = C.c_void_p
    lib.rbv_symm_alloc.argtypes = [C.c_void_p, C.c_size_t]
    lib.rbv_symm_free.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_in_heap.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    lib.rbv_comm.restype = C.c_void_p
    lib.rbv_comm.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_comm_rank.argtypes = [C.c_void_p]
    lib.rbv_comm_size.argtypes = [C.c_void_p]
    lib.rbv_alltoallv.argtypes = [C.c_void_p] + [C.c_int] * 7 + [
        C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
        C.c_int, C.c_longlong, C.c_uint, C.c_int, C.c_size_t, C.c_void_p]
    lib.rbv_update_timers.argtypes = [C.c_void_p]
    lib.rbv_prepare.restype = C.c_void_p
    lib.rbv_prepare.argtypes = [C.c_void_p] + [C.c_int] * 7 + [
        C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
        C.c_int, C.c_longlong, C.c_uint, C.c_int, C.c_size_t]
    lib.rbv_prepare_global.restype = C.c_void_p
    lib.rbv_prepare_global.argtypes = lib.rbv_prepare.argtypes + [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.rbv_prepared_info.argtypes = [C.c_void_p, c_ll_p]
    lib.rbv_ctx_set_static.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_ctx_set_recv_mirror.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_set_recv_mirror.restype = None
    lib.rbv_ctx_last_trace.argtypes = [C.c_void_p, C.POINTER(C.c_uint), C.POINTER(C.c_ulonglong),
                                       C.POINTER(C.c_ulonglong), C.c_int]
    lib.rbv_iteration_count.argtypes = [C.c_void_p]
    lib.rbv_ctx_set_auto_hint.argtypes = [C.c_void_p, C.c_double, C.c_double]
    lib.rbv_ctx_last_choice.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.rbv_prepared_free.argtypes = [C.c_void_p, C.c_void_p]
    lib.rbv_ctx_set_trace.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_ctx_set_bulk.argtypes = [C.c_void_p, C.c_int]
    lib.rbv_ctx_set_nvls_meta.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
    lib.rbv_ctx_meta_bytes.restype = C.c_size_t
    lib.rbv_ctx_meta_bytes.argtypes = [C.c_void_p]
    lib.rbv_ctx_nvls_create.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
    lib.rbv_ctx_nvls_import.argtypes = [C.c_void_p, C.c_int, C.c_size_t]
    lib.rbv_ctx_nvls_add_device.argtypes = [C.c_void_p]
    lib.rbv_ctx_nvls_bind.argtypes = [C.c_void_p]
    lib.rbv_ctx_nvls_teardown.argtypes = [C.c_void_p]
    lib.rbv_ctx_set_eager.argtypes = [C.c_void_p, C.c_ulonglong]
    lib.rbv_ctx_set_cooperative.argtypes = [C.c_void_p, C.c_int]
    declare_moe(lib)
    lib.rbv_alltoallv_noalloc.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.rbv_noalloc_status.argtypes = [C.c_void_p]
    lib.rbv_noalloc_last_error.restype = C.c_char_p
    lib.rbv_transpose_exchange.argtypes = [C.c_void_p, C.c_void_p, C.c_ulonglong, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_int, C.c_void_p]


def declare_moe(lib):
    vp, i, ll, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_ulonglong
    lib.rbv_grouped_gemm_bf16.argtypes = [vp, ll, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_bf16_pair.argtypes = [vp, ll, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_set_pair.argtypes = [i]
    lib.rbv_grouped_gemm_set_pair.restype = None
    lib.rbv_grouped_gemm_pair_enabled.argtypes = []
    lib.rbv_grouped_gemm_fp8.argtypes = [vp, vp, ll, vp, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_fp8_pair.argtypes = [vp, vp, ll, vp, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_mxfp8.argtypes = [vp, vp, ll, vp, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_mxfp8_swiglu_q.argtypes = [vp, vp, ll, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, i, vp]
    lib.rbv_grouped_gemm_bf16_push.argtypes = [vp, ll, vp, vp, vp, i, i, i, vp, vp, i, ull, vp, i, vp]
    lib.rbv_grouped_gemm_mxfp8_push.argtypes = [vp, vp, ll, vp, vp, vp, vp, i, i, i, vp, vp, i, ull, vp, i, vp]
    lib.rbv_moe_dispatch_ret.argtypes = [vp, vp, i, i, vp, vp, vp, vp, ull, ull, ll, i, vp, vp]
    lib.rbv_moe_dispatch_mx.argtypes = [vp, vp, i, i, vp, vp, vp, vp, ull, ull, ull, ll, i, vp, vp]
    lib.rbv_moe_scale_atoms.argtypes = [vp, vp, i, i, vp]
    lib.rbv_moe_combine_pushed.argtypes = [vp, vp, i, i, vp, vp, vp, vp]
    lib.rbv_quantize_rows_mxfp8.argtypes = [vp, ll, i, i, vp, vp, vp]
    lib.rbv_quantize_rows_fp8.argtypes = [vp, ll, i, i, vp, vp, vp]
    lib.rbv_moe_route.argtypes = [vp, i, i, vp, vp, vp, vp]
    lib.rbv_moe_layout.argtypes = [vp, i, i, i, vp, vp, vp, vp, vp, vp]
    lib.rbv_moe_layout_aligned.argtypes = [vp, i, i, i, vp, vp, vp, vp, vp, i, vp]
    lib.rbv_moe_layout_streamed.argtypes = [vp, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp, i, vp, vp]
    lib.rbv_moe_dispatch_streamed.argtypes = [vp, vp, i, i, vp, vp, vp, vp, vp, ull, ull, ll, i, vp, vp]
    lib.rbv_grouped_gemm_bf16_gated.argtypes = [vp, ll, vp, vp, vp, vp, i, i, i, i, i, vp, i, vp, vp, vp, C.c_double]
    lib.rbv_moe_dispatch.argtypes = [vp, vp, i, i, vp, vp, vp, vp, ull, ll, i, vp, vp]
    lib.rbv_moe_combine.argtypes = [vp, vp, i, i, vp, vp, vp, ull, i, vp, vp]
