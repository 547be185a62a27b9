"""spion_b200: B200-native implementation of SPION's layer-wise block-sparse attention path.

Importing the package does not load CUDA code; the submodules that call the native library
(``pattern``, ``attention*``, ``native``) import ``spion_b200._lib``, which raises if
``spion_b200/lib/libspion_b200.so`` has not been built.  There is no CPU fallback.
"""
__version__ = "0.1.0"
