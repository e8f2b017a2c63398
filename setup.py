"""Packaging of ``torchrec_b200``.  The CUDA (sm_100a) and host C++ extensions are built in-tree by
``python -c "import __graft_entry__ as g; g.build()"`` (or ``python -m torchrec_b200.csrc.build``) before ``pip install .``; the
built shared objects travel as package data."""
import os

from setuptools import find_packages, setup

here = os.path.dirname(os.path.abspath(__file__))
about = {}
with open(os.path.join(here, "torchrec_b200", "version.py")) as f:
    exec(f.read(), about)

setup(
    name="torchrec_b200",
    version=about["__version__"],
    description="Blackwell-native sharded-embedding recommender framework",
    long_description=open(os.path.join(here, "README.md")).read(),
    long_description_content_type="text/markdown",
    packages=find_packages(include=["torchrec_b200", "torchrec_b200.*"]),
    package_data={"torchrec_b200": ["*.so", "csrc/cuda/*.cu", "csrc/cuda/*.h", "csrc/cuda/*.cuh", "csrc/cpu/*.cpp", "csrc/cpu/*.h", "csrc/cpu/plugins/*.cpp",
                                    "csrc/cpu/tests/*.cpp", "distributed/benchmark/yaml/*.yml"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pyyaml", "tqdm"],
    extras_require={"serving": ["grpcio", "protobuf"], "test": ["pytest", "hypothesis", "scikit-learn"]},
    zip_safe=False,
)
