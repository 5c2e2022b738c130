"""B200-native VDCores decode runtime: a persistent sm_100a megakernel driven by
per-SM memory/compute instruction streams, behind a C ABI (include/vdcores.h)."""
__version__ = "0.1.0"
