"""Helpers around the native library: configuration files, device timing, clock
sampling, the operator CLI."""
