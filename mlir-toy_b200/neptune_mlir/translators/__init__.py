"""HTile translators.  ``b200`` is the only target: hand-written sm_100a kernels behind a C ABI."""
