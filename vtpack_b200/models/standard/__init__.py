"""Counterparts of ``vtpack/models/standard``: the parts that call this library's native ops."""
