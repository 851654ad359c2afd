"""Shipped agent presets, one file each: ``<name>_<id>_<parent id>.py`` exporting ``config``."""
