//! Raw declarations of `include/datago_b200.h`, one for one.  Written for datago's workers
//! (`src/worker_files.rs`, `src/worker_wds.rs`, `src/worker_http.rs`), which today call
//! `image::load_from_memory` + `image_processing::image_to_payload` per sample; see INTEGRATION.md for the call sites.
//! Not compiled in the repository's build container (no Rust toolchain there); the same C ABI is exercised by the
//! ctypes binding in `datago_b200/__init__.py`.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

pub const DG_OK: c_int = 0;
pub const DG_E_INVALID: c_int = 1;
pub const DG_E_CUDA: c_int = 2;
pub const DG_E_TRUNCATED: c_int = 3;
pub const DG_E_BAD_MARKER: c_int = 4;
pub const DG_E_UNSUPPORTED: c_int = 5;
pub const DG_E_BAD_TABLE: c_int = 6;
pub const DG_E_BAD_CODE: c_int = 7;
pub const DG_E_UNKNOWN_KEY: c_int = 8;
pub const DG_E_NO_TRANSFORM: c_int = 9;
pub const DG_E_SYNC_LIMIT: c_int = 10;
pub const DG_E_TOO_LARGE: c_int = 11;
pub const DG_E_TIMEOUT: c_int = 12;
pub const DG_STATUS_COUNT: usize = 13;

pub const DG_DEVICE_NONE: c_int = -1;
pub const DG_ITEM_TO_RGB8: u32 = 1;
pub const DG_BATCH_DECODE_ONLY: u32 = 1;
pub const DG_BATCH_TIMING: u32 = 2;
pub const DG_BATCH_KEEP_COEFFICIENTS: u32 = 4;
pub const DG_BATCH_COLLATE: u32 = 8;
pub const DG_STAGE_COUNT: usize = 10;
pub const DG_LOG_ERROR: c_int = 1;
pub const DG_LOG_WARN: c_int = 2;

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dg_image_config {
    pub crop_and_resize: i32,
    pub default_image_size: u32,
    pub downsampling_ratio: u32,
    pub min_aspect_ratio: f64,
    pub max_aspect_ratio: f64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dg_plan {
    pub src_w: u32,
    pub src_h: u32,
    pub channels: u32,
    pub target_w: u32,
    pub target_h: u32,
    pub new_w: u32,
    pub new_h: u32,
    pub crop_left: f64,
    pub crop_top: f64,
    pub crop_w: f64,
    pub crop_h: f64,
    pub identity: i32,
    pub key: [c_char; 16],
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dg_jpeg_info {
    pub width: u32,
    pub height: u32,
    pub channels: u32,
    pub hsamp: u32,
    pub vsamp: u32,
    pub mcux: u32,
    pub mcuy: u32,
    pub restart_interval: u32,
    pub scan_offset: u64,
    pub scan_len: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct dg_item {
    pub data: *const u8,
    pub len: u64,
    pub raw_w: u32,
    pub raw_h: u32,
    pub raw_c: u32,
    pub flags: u32,
    pub forced_key: *const c_char,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct dg_result {
    pub status: i32,
    pub original_width: u32,
    pub original_height: u32,
    pub width: u32,
    pub height: u32,
    pub channels: u32,
    pub bit_depth: u32,
    pub nbytes: u64,
    pub device_data: *const u8,
    pub plan: dg_plan,
    pub packed_offset: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct dg_bucket {
    pub key: [c_char; 16],
    pub n: u32,
    pub width: u32,
    pub height: u32,
    pub channels: u32,
    pub nbytes: u64,
    pub device_data: *const u8,
    pub packed_offset: u64,
    pub items: *const i32,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct dg_feeder_config {
    pub lanes: u32,
    pub max_batch: u32,
    pub max_wait_us: u32,
    pub queue_limit: u32,
    pub batch_flags: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Default, Debug)]
pub struct dg_feeder_stats {
    pub submitted: u64,
    pub completed: u64,
    pub failed: u64,
    pub batches: u64,
    pub batched_items: u64,
    pub largest_batch: u32,
    pub queued: u32,
    pub open_tickets: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct dg_ctx_counters {
    pub items: [u64; DG_STATUS_COUNT],
    pub batches: u64,
    pub bytes_in: u64,
    pub bytes_out: u64,
}

pub enum dg_ctx {}
pub enum dg_batch {}
pub enum dg_feeder {}
pub type dg_ticket = u64;
pub type dg_log_fn = Option<unsafe extern "C" fn(level: c_int, message: *const c_char, user: *mut c_void)>;

extern "C" {
    pub fn dg_last_error() -> *const c_char;
    pub fn dg_version() -> *const c_char;
    pub fn dg_set_log_callback(f: dg_log_fn, user: *mut c_void);

    pub fn dg_ctx_create(device: c_int, cfg: *const dg_image_config, out: *mut *mut dg_ctx) -> c_int;
    pub fn dg_ctx_create_on_stream(device: c_int, cfg: *const dg_image_config, cuda_stream: *mut c_void, out: *mut *mut dg_ctx) -> c_int;
    pub fn dg_ctx_destroy(ctx: *mut dg_ctx);
    pub fn dg_ctx_stream(ctx: *mut dg_ctx) -> *mut c_void;
    pub fn dg_ctx_get_counters(ctx: *mut dg_ctx, out: *mut dg_ctx_counters) -> c_int;

    pub fn dg_size_list(cfg: *const dg_image_config, max_n: c_int, w: *mut u32, h: *mut u32) -> c_int;
    pub fn dg_bucket_table(ctx: *const dg_ctx, max_n: c_int, w: *mut u32, h: *mut u32, ar: *mut f64, keys: *mut c_char) -> c_int;
    pub fn dg_closest_aspect_ratio(ctx: *const dg_ctx, w: i32, h: i32, key_out: *mut c_char) -> c_int;
    pub fn dg_aspect_ratio_to_str(w: u32, h: u32, key_out: *mut c_char);
    pub fn dg_plan_geometry(ctx: *const dg_ctx, w: u32, h: u32, channels: u32, forced_key: *const c_char, out: *mut dg_plan) -> c_int;
    pub fn dg_jpeg_probe(data: *const u8, len: u64, out: *mut dg_jpeg_info) -> c_int;

    pub fn dg_rank_slice(quorum: u64, rank: u64, world_size: u64, start: *mut u64, end: *mut u64) -> c_int;
    pub fn dg_key_hash(key: *const c_char, len: u64) -> u64;
    pub fn dg_key_rank(key: *const c_char, len: u64, world_size: u64) -> u64;

    pub fn dg_batch_create(ctx: *mut dg_ctx, items: *const dg_item, n: c_int, flags: u32, out: *mut *mut dg_batch) -> c_int;
    pub fn dg_batch_upload(b: *mut dg_batch) -> c_int;
    pub fn dg_batch_run(b: *mut dg_batch) -> c_int;
    pub fn dg_batch_download(b: *mut dg_batch, host_out: *const *mut u8) -> c_int;
    pub fn dg_batch_download_packed(b: *mut dg_batch, host_base: *mut u8, capacity: u64) -> c_int;
    pub fn dg_batch_packed_bytes(b: *const dg_batch) -> u64;
    pub fn dg_batch_sync(b: *mut dg_batch) -> c_int;
    pub fn dg_batch_result(b: *const dg_batch, i: c_int, out: *mut dg_result) -> c_int;
    pub fn dg_batch_bucket_count(b: *const dg_batch) -> c_int;
    pub fn dg_batch_bucket(b: *const dg_batch, k: c_int, out: *mut dg_bucket) -> c_int;
    pub fn dg_batch_stage_ms(b: *const dg_batch, ms: *mut f32) -> c_int;
    pub fn dg_batch_counters(b: *const dg_batch, h2d_bytes: *mut u64, d2h_bytes: *mut u64, kernel_launches: *mut u32) -> c_int;
    pub fn dg_batch_huffman_stats(b: *mut dg_batch, out: *mut u64) -> c_int;
    pub fn dg_batch_debug(b: *const dg_batch, i: c_int, coef: *mut *const i16, nblocks: *mut u64, decoded: *mut *const u8) -> c_int;
    pub fn dg_batch_destroy(b: *mut dg_batch);
    pub fn dg_process(ctx: *mut dg_ctx, items: *const dg_item, n: c_int, flags: u32, host_out: *const *mut u8, results: *mut dg_result) -> c_int;

    pub fn dg_feeder_create(device: c_int, image_config: *const dg_image_config, config: *const dg_feeder_config, out: *mut *mut dg_feeder) -> c_int;
    pub fn dg_feeder_ctx(f: *const dg_feeder) -> *const dg_ctx;
    pub fn dg_submit(f: *mut dg_feeder, item: *const dg_item, host_out: *mut u8, host_capacity: u64, ticket: *mut dg_ticket) -> c_int;
    pub fn dg_wait(f: *mut dg_feeder, ticket: dg_ticket, timeout_ns: u64, out: *mut dg_result) -> c_int;
    pub fn dg_fetch(f: *mut dg_feeder, ticket: dg_ticket, host_out: *mut u8, capacity: u64) -> c_int;
    pub fn dg_peek(f: *mut dg_feeder, ticket: dg_ticket, host_data: *mut *const u8) -> c_int;
    pub fn dg_release(f: *mut dg_feeder, ticket: dg_ticket) -> c_int;
    pub fn dg_feeder_get_stats(f: *mut dg_feeder, out: *mut dg_feeder_stats) -> c_int;
    pub fn dg_feeder_destroy(f: *mut dg_feeder);

    pub fn dg_resize_device_static(ctx: *mut dg_ctx, device_src: *const u8, w: u32, h: u32, channels: u32, forced_key: *const c_char,
                                   device_dst: *mut u8, plan_out: *mut dg_plan) -> c_int;
    pub fn dg_copy_to_host(ctx: *mut dg_ctx, dst: *mut c_void, device_src: *const c_void, nbytes: u64) -> c_int;
}
