"""Packaging for dion_b200.  The CUDA extension is built in-tree for sm_100a by
`python -c "import __graft_entry__ as g; g.build()"` (or dion_b200.ops._ext.build())."""
from setuptools import find_packages, setup

setup(
    name="dion_b200",
    version="0.1.0",
    description="Blackwell-native Dion / Muon optimizers and GPT training stack",
    packages=find_packages(include=["dion_b200", "dion_b200.*"]),
    package_data={"dion_b200": ["csrc/*", "_C/*.so"]},
    python_requires=">=3.10",
    install_requires=["numpy", "torch>=2.7.1", "pyyaml"],
    extras_require={"dev": ["pytest", "pytest-timeout"], "train": ["huggingface-hub", "wandb", "datasets", "tiktoken", "tqdm"]},
)
