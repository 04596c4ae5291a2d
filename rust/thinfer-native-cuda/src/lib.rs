//! Bindings of the NVFP4 linear path for B200. `ffi` is generated from include/thinfer_nvfp4.h
//! (gen_ffi.py). Link against thinfer_b200/libthinfer_nvfp4.so. Not compiled in this repository's
//! own checks (no Rust toolchain in its build image): tests/test_abi.py checks the symbol list and
//! the struct sizes against the header instead.
pub mod ffi;

use std::os::raw::c_void;

/// The blocking core of `WeightReader` (thinfer-core/src/weight.rs:57-77) that the library's chunk
/// loops drive. An async reader is adapted by blocking on its future inside `read_at`.
pub trait BlockingReader {
    fn len(&self) -> u64;
    fn read_at(&mut self, offset: u64, dst: &mut [u8]) -> Result<(), String>;
    fn will_read(&mut self, _offset: u64, _len: u64) {}
}

unsafe extern "C" fn reader_len<R: BlockingReader>(user: *mut c_void) -> u64 {
    (*(user as *mut R)).len()
}

unsafe extern "C" fn reader_read_at<R: BlockingReader>(user: *mut c_void, offset: u64, dst: *mut c_void, n: u64) -> i32 {
    let dst = std::slice::from_raw_parts_mut(dst as *mut u8, n as usize);
    match (*(user as *mut R)).read_at(offset, dst) {
        Ok(()) => ffi::TNF_OK,
        Err(_) => ffi::TNF_ERR_INVALID_ARGUMENT,
    }
}

unsafe extern "C" fn reader_will_read<R: BlockingReader>(user: *mut c_void, offset: u64, n: u64) {
    (*(user as *mut R)).will_read(offset, n)
}

unsafe extern "C" fn reader_close<R: BlockingReader>(user: *mut c_void) {
    drop(Box::from_raw(user as *mut R));
}

/// Hands a reader to the library: `tnf_reader_read`, `tnf_reader_read_to_arena` and
/// `tnf_upload_from_reader` call back into it. `ffi::tnf_reader_close` drops the box.
pub fn reader_for<R: BlockingReader>(reader: Box<R>) -> ffi::TnfReader {
    ffi::TnfReader {
        user: Box::into_raw(reader) as *mut c_void,
        len: Some(reader_len::<R>),
        read_at: Some(reader_read_at::<R>),
        will_read: Some(reader_will_read::<R>),
        close: Some(reader_close::<R>),
    }
}
