"""torchrun entry point: ``torchrun --standalone --nproc_per_node=N train.py --config configs/dion_160m.yaml``
(same command line and YAML keys as the reference's train.py:85-224, 582-959; the code is in
``dion_b200/training.py``)."""
from dion_b200.training import main

if __name__ == "__main__":
    main()
