"""Architectures this package knows; importing the package registers them."""

from oxr_inference_b200.models import bifusun, nidudra, qwen3, radapel, vazepel  # noqa: F401
