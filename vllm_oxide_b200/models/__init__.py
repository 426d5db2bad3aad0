"""Architectures this engine knows. Importing the package registers them."""
from .llama import LLAMA, BuildContext, build_llama, llama_manifest
from .rotepel import ROTEPEL, build_rotepel, rotepel_manifest
from .lomopel import LOMOPEL, build_lomopel, lomopel_manifest
from .bufulorn import BUFULORN, build_bufulorn, bufulorn_manifest
from .pironex import PIRONEX, build_pironex, pironex_manifest

__all__ = ["LLAMA", "BuildContext", "build_llama", "llama_manifest", "ROTEPEL", "build_rotepel", "rotepel_manifest",
           "LOMOPEL", "build_lomopel", "lomopel_manifest", "BUFULORN", "build_bufulorn", "bufulorn_manifest",
           "PIRONEX", "build_pironex", "pironex_manifest"]
