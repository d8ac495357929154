import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def native_built():
    """Build (if stale) and return the paths of the native libraries. Device-side waits are
    given a short limit for the test session, so a kernel that stalls fails in well under a
    second per launch instead of holding the GPU."""
    from b200_attention_b200 import _native, build

    built = build.build_all()
    _native.lib().b200attn_set_wait_limit_ms(400)
    return built
