"""Test-support code that ships with the package (pytest plugins)."""
