import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library and the CPU checker are built once per session (both build without a GPU)."""
    from codegendemo_b200 import build as kbuild
    from oracle import build_oracle
    kbuild.build_library()
    build_oracle.build_port()
    yield


@pytest.fixture()
def work_dir(tmp_path):
    from codegendemo_b200.kcg.Utils import PathManager
    old = PathManager._root
    PathManager.set_project_dir(str(tmp_path / "kcg_work"))
    PathManager.init()
    yield str(tmp_path / "kcg_work")
    PathManager._root = old
    os.environ.pop("KCG_WORK_DIR", None)
