"""B200-native (sm_100a) low-precision linear path: quantizers, scaled / block-scaled GEMMs and
the MoE data movement, behind the call signatures of gongyisheng/pretrain's ``src/quant``."""

__all__ = ["ops"]
