"""Compute tiles: host runners with the reference's signatures over libmdc.so."""
