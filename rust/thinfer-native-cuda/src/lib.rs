//! Bindings of the NVFP4 linear path for B200. `ffi` is generated from include/thinfer_nvfp4.h
//! (gen_ffi.py). Link against thinfer_b200/libthinfer_nvfp4.so. Not compiled in this repository's
//! own checks (no Rust toolchain in its build image): tests/test_abi.py checks the symbol list and
//! the struct sizes against the header instead.
pub mod ffi;
