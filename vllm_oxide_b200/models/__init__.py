"""Architectures this engine knows. Importing the package registers them."""
from .llama import LLAMA, BuildContext, build_llama, llama_manifest

__all__ = ["LLAMA", "BuildContext", "build_llama", "llama_manifest"]
