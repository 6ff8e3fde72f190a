"""Mirrors of the reference's moe/ modules backed by libb200moe.so."""
