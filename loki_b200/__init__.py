"""loki_b200: B200-native exact vector scan behind the API of Lowkey Media Server's
``embedindex`` / ``embedvec`` packages.

* ``loki_b200.embedindex``  path-keyed index with the reference's interface
  (``New``, ``NewCentered``, ``Add``, ``Delete``, ``Search*``, ``Len``)
* ``loki_b200._lib``        ctypes binding of the C ABI in ``include/lokiscan.h``
* ``loki_b200.build``       compiles ``liblokiscan.so`` in-tree

Everything computes on the GPU through ``liblokiscan.so``; there is no CPU path.
Importing ``_lib`` or ``embedindex`` raises if the library has not been built.
"""
__version__ = "0.1.0"
__all__ = ["embedindex", "embedvec", "_lib", "build"]


def __getattr__(name):
    if name in ("embedindex", "embedvec", "_lib", "build"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
