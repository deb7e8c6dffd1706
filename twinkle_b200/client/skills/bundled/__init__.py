"""Markdown skills shipped with the package."""
