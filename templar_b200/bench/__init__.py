"""Benchmarks of the secondary configurations (the headline one is ``bench.py`` at the repository root):
``config3_gather`` (compressed-gradient gather), ``config4_tp`` (18B-class tensor-parallel window) and
``config5_validator`` (validator scoring).  Each prints one JSON line per case."""
