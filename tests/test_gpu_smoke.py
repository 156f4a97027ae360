import pytest

pytestmark = pytest.mark.gpu


def test_extension_is_loaded():
    from torchure_b200 import ops

    assert ops.available(), "the sm_100a extension must be the code path on a GPU box"
