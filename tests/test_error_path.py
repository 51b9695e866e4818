"""A non-zero status from a C entry point must surface as a Python exception (it used to end the
process with SIGSEGV).  Runs without a GPU: the op only formats and raises."""
import pytest
import torch


def test_status_codes_raise_instead_of_crashing():
    from warpstate_ai_b200.ops import _ext
    if not _ext.load():
        pytest.skip("kernel library not built")
    assert torch.ops.ws_b200.raise_for_status(0) == 0
    for code in (-1, -11, -21):
        with pytest.raises(RuntimeError, match=f"failed with code {code}"):
            torch.ops.ws_b200.raise_for_status(code)
