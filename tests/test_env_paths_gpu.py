"""The library's alternative code paths (environment variables read once per process)
give the same results as the defaults: a child process per setting runs
env_paths_worker.py against the CPU oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("env", [{}, {"B200_PDL": "0", "B200_WALK_RING": "0", "B200_GRID_WAVES": "1"}],
                         ids=["defaults", "serialised_register_walk_one_wave"])
def test_env_paths(env):
    p = subprocess.run([sys.executable, os.path.join(HERE, "env_paths_worker.py")], env=dict(os.environ, **env),
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:]
    assert "ENV_PATHS_OK" in p.stdout
