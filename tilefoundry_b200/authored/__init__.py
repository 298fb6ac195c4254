"""Signature-level declarations of the authored Modules whose decode step this
library implements (one file per model), plus seeded synthetic weights."""
