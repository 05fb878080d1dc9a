"""Packaging: the project installs from its pyproject.toml (no index, no build isolation) with its
CUDA sources and shape files as package data and its two console scripts, and the installed copy
runs from another working directory (mini_hisparse's own: pyproject.toml:34-38)."""
import os
import shutil
import subprocess
import sys
import tomllib

import pytest

from conftest import ROOT


def test_console_scripts_point_at_functions():
    meta = tomllib.loads((ROOT / "pyproject.toml").read_text())
    scripts = meta["project"]["scripts"]
    assert set(scripts) == {"mini-hisparse-b200", "trace_run"}
    for target in scripts.values():
        module, func = target.split(":")
        assert callable(getattr(__import__(module, fromlist=[func]), func))


@pytest.fixture(scope="module")
def installed(tmp_path_factory):
    target = tmp_path_factory.mktemp("site")
    # from a copy of the sources: a build leaves build/ and .egg-info folders beside what it builds
    source = tmp_path_factory.mktemp("source")
    for name in ("pyproject.toml", "README.md"):
        shutil.copy(ROOT / name, source / name)
    shutil.copytree(ROOT / "mini_hisparse_b200", source / "mini_hisparse_b200",
                    ignore=shutil.ignore_patterns("_build", "__pycache__"))
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
           "--target", str(target), str(source)]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=tmp_path_factory.mktemp("elsewhere"))
    if proc.returncode != 0:
        pytest.skip(f"pip could not build the project offline here: {proc.stderr[-400:]}")
    return target


def test_installed_copy_has_sources_shapes_and_scripts(installed):
    pkg = installed / "mini_hisparse_b200"
    for name in ("gemm_tc.cu", "attention_decode.cu", "common.cuh", "gemm_simt_noalloc.h"):
        assert (pkg / "csrc" / name).exists(), name
    assert (pkg / "configs" / "qwen2.5-7b-shape.json").exists() and (pkg / "configs" / "demo.json").exists()
    assert not list((pkg / "csrc").glob("_build/*.so")), "built libraries must not be packaged"
    assert (installed / "bin" / "mini-hisparse-b200").exists() and (installed / "bin" / "trace_run").exists()


def test_installed_command_line_runs_from_another_folder(installed, tmp_path):
    """Without a GPU the commands still parse their options and say what is missing."""
    env = dict(os.environ, PYTHONPATH=str(installed))
    for script, args in (("mini-hisparse-b200", ["demo", "--help"]), ("trace_run", ["--help"])):
        proc = subprocess.run([sys.executable, str(installed / "bin" / script), *args], capture_output=True, text=True,
                              cwd=tmp_path, env=env)
        assert proc.returncode == 0 and "usage" in proc.stdout.lower(), proc.stderr
    probe = ("import mini_hisparse_b200, pathlib; p = pathlib.Path(mini_hisparse_b200.__file__).parent; "
             "print(p); from mini_hisparse_b200.kernels import build; print(build.CSRC)")
    proc = subprocess.run([sys.executable, "-c", probe], capture_output=True, text=True, cwd=tmp_path, env=env)
    assert proc.returncode == 0 and str(installed) in proc.stdout, proc.stderr


@pytest.mark.gpu
def test_installed_copy_generates(installed, tmp_path):
    """The installed copy, from another folder: its kernels compile into a folder it can write and the
    demo generates tokens."""
    env = dict(os.environ, PYTHONPATH=str(installed), MHB200_BUILD_DIR=str(tmp_path / "build"))
    proc = subprocess.run([sys.executable, str(installed / "bin" / "mini-hisparse-b200"), "demo", "--requests", "2",
                           "--prompt-tokens", "20", "--max-new-tokens", "4", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=tmp_path, env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert '"outputs"' in proc.stdout
