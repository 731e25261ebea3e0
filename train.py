"""torchrun entry point: ``torchrun --standalone --nproc_per_node=N train.py --config configs/dion_160m.yaml``."""
from dion_b200.training import main

if __name__ == "__main__":
    main()
