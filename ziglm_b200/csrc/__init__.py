from .builder import KernelBuildError, build, library_path, load, sources

__all__ = ["KernelBuildError", "build", "library_path", "load", "sources"]
