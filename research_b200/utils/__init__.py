"""Utilities: device timing, logging, config loading, fingerprints, tensor rendering."""
