"""Token-level sparse attention kernels (B200 build).

Same layout as the reference's ``mcsparse.kernels``: submodules are not imported at
package load time, so pure-logic code works without PyTorch or the shared library.
"""

__version__ = "0.1.0"

__all__: list[str] = []
