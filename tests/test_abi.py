"""The C-ABI shared library loads on a machine without a GPU and exports every
function the public headers declare (no compute call is made here)."""
import ctypes as C
import importlib
import os

import pytest

pkg = importlib.import_module("jdm-ghassan_v1_flach_b200")
capi = importlib.import_module("jdm-ghassan_v1_flach_b200.capi")


@pytest.fixture(scope="module")
def so():
    assert os.path.exists(capi.LIB_PATH), "libb200ops.so is not built (run __graft_entry__.build())"
    return C.CDLL(capi.LIB_PATH)


def test_headers_declare_the_reference_surface():
    names = set(capi.declared_symbols())
    # one entry point per reference op on the hot path, plus the decoder and the quantisers
    for must in ("b200_linear_forward_q4", "b200_linear_forward_fp16", "b200_linear_forward_f32",
                 "b200_dequantize_quant", "b200_embedding_forward_half", "b200_rmsnorm_forward",
                 "b200_rope_forward_cached", "b200_swiglu_forward", "b200_moe_forward_bias_half",
                 "b200_moe_permutation", "b200_mamba2_forward_half", "b200_mamba2_step_half",
                 "b200_attention_forward_ex", "b200_attention_decode_ring_fp16", "b200_topk_select",
                 "b200_argmax_token", "b200_apply_rep_penalties", "b200_decoder_create",
                 "b200_decoder_step_host", "b200_quantize", "b200_last_error"):
        assert must in names, must
    assert len(names) > 80


def test_every_declared_symbol_is_exported(so):
    missing = [n for n in capi.declared_symbols() if not hasattr(so, n)]
    assert not missing, missing


def test_version_and_error_string(so):
    so.b200_last_error.restype = C.c_char_p
    assert so.b200_version() > 0
    assert isinstance(so.b200_last_error(), bytes)


def test_argument_errors_are_status_codes_not_aborts(so):
    """Validation happens before any device work, so it is observable without a GPU."""
    so.b200_last_error.restype = C.c_char_p
    rc = so.b200_linear_forward_q4(None, None, None, 1, 33, 4, 0)       # K % 32 != 0
    assert rc < 0
    assert so.b200_last_error()
    rc = so.b200_training_op_unsupported(b"adamw_step")
    assert rc < 0 and b"adamw_step" in so.b200_last_error()


def test_python_binding_fails_loudly_without_the_library(tmp_path):
    with pytest.raises(OSError, match="no CPU or PyTorch fallback"):
        capi.Library(str(tmp_path / "absent.so"))


def test_value_returning_functions_do_not_raise():
    """b200_version and the gemm toggles' getters return values, not status codes: the
    Python binding must hand them back instead of raising on a non-zero result."""
    lib = pkg.lib()
    assert lib.b200_version() == 100
    assert lib.b200_fp16_gemm_enabled() in (0, 1)
    assert "b200_version" in capi.VALUE_RETURNING
