"""setuptools entry for the B200 build: `python setup.py build_ext --inplace` compiles libfda_sm100.so with nvcc
for sm_100a only (the reference's setup.py:114 builds for sm_90a only). The heavy lifting is in build_lib.py."""

import os
import sys

from setuptools import Command, setup

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

exec(open(os.path.join(HERE, "fast_diffusion_attention", "version.py")).read())


class BuildLib(Command):
    description = "compile libfda_sm100.so in-tree with nvcc (sm_100a)"
    user_options = [("inplace", "i", "kept for `build_ext --inplace` compatibility"), ("force", "f", "rebuild all")]

    def initialize_options(self):
        self.inplace = 1
        self.force = 0

    def finalize_options(self):
        pass

    def run(self):
        if os.environ.get("FDA_SKIP_CUDA_BUILD", "0") == "1":
            return
        import build_lib
        print(build_lib.build(force=bool(self.force), verbose=True))


setup(
    name="fast_diffusion_attention",
    version=__version__,  # noqa: F821
    packages=["fast_diffusion_attention"],
    package_data={"fast_diffusion_attention": ["libfda_sm100.so"]},
    cmdclass={"build_ext": BuildLib},
    python_requires=">=3.9",
)
