"""HTile front end and translators with a B200-native (sm_100a) CUDA target.

Mirrors the package layout of the reference (src/neptune_mlir): ``plugin`` locates native
libraries, ``translators`` holds one module per target.  The only target here is
``translators.b200``, which lowers an HTile program to calls into the nb200 kernel library.
"""

__version__ = "0.1.0"
