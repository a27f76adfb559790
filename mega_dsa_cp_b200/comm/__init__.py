"""Comm layer: symmetric payload arena and the device-side peer view."""
