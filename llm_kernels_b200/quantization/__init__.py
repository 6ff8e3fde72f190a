"""Mirrors of the reference's quantization/ modules backed by libb200moe.so."""
