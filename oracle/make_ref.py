"""Stage the unmodified reference package beside the oracle (test and baseline infrastructure).

    python oracle/make_ref.py <reference checkout>

installs the reference's own project (``projects/gl-sdm`` of the checkout, pure Python) with
pip into ``oracle/_ref/`` - offline, without its dependencies, from a scratch copy because
the build writes into the source tree. ``oracle/_ref/`` is ignored by git, so no reference
source enters the history; a working tree that holds it can import ``gl_sdm`` from there on a
machine that has no checkout. Only tests, ``bench.py --impl reference`` / ``cpu_baseline``
and ``__graft_entry__.build()`` use it; nothing under ``gl_sdm_b200/`` may import it.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
PROJECT = os.path.join("projects", "gl-sdm")


def ref_path():
    """Directory to put on sys.path to import the staged reference, or None."""
    return TARGET if os.path.exists(os.path.join(TARGET, "gl_sdm", "__init__.py")) else None


def stage(checkout, force=False):
    """Install <checkout>/projects/gl-sdm into oracle/_ref. Returns the target directory."""
    project = os.path.join(checkout, PROJECT)
    if not os.path.exists(os.path.join(project, "pyproject.toml")):
        raise FileNotFoundError(f"no reference project at {project}")
    if ref_path() and not force:
        return TARGET
    with tempfile.TemporaryDirectory() as scratch:
        source = os.path.join(scratch, "gl-sdm")
        shutil.copytree(project, source, ignore=shutil.ignore_patterns("results", "__pycache__", ".git"))
        staged = os.path.join(scratch, "target")
        command = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation",
                   "--no-deps", "--target", staged, source]
        done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if done.returncode != 0:
            raise RuntimeError("pip could not install the reference:\n" + done.stdout[-2000:])
        if os.path.exists(TARGET):
            shutil.rmtree(TARGET)
        shutil.copytree(staged, TARGET, ignore=shutil.ignore_patterns("__pycache__", "bin"))
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(stage(sys.argv[1], force=True))
