"""Build hook: the public header lives in ``include/`` at the repository root; an installed copy of
the package carries it beside the CUDA sources so that ``flyvec_compile`` still finds it."""
import shutil
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


class build_py_with_header(build_py):
    def run(self):
        super().run()
        root = Path(__file__).resolve().parent
        dst = Path(self.build_lib) / "flyvec_b200" / "csrc"
        dst.mkdir(parents=True, exist_ok=True)
        for h in (root / "include").glob("*.h"):
            shutil.copy2(h, dst / h.name)


setup(cmdclass={"build_py": build_py_with_header})
