"""B200-native post-training framework: SFT, DPO, GRPO/RLVR and reward modelling on
hand-written sm_100a kernels with NVLink-fused collectives."""

__version__ = "0.1.0"
