//! Raw bindings for `include/xlb.h` (module `ffi`) and a safe layer over them (module `safe`).
//!
//! Not compiled in the repository this file ships in: there is no Rust toolchain in its build
//! image.  Field order, widths and constants follow `include/xlb.h` line by line.
#![allow(non_camel_case_types)]

pub mod ffi {
    use std::os::raw::{c_char, c_int, c_void};

    pub const XLB_MAX_ARITY: usize = 8;
    pub const XLB_MAX_KEYS: usize = 2;
    pub const XLB_UNIQUE_ID_BYTES: usize = 128;

    // xlb_status
    pub const XLB_OK: c_int = 0;
    pub const XLB_ERR_INVALID: c_int = 1;
    pub const XLB_ERR_TYPE: c_int = 2;
    pub const XLB_ERR_RESOURCE_EXHAUSTED: c_int = 3;
    pub const XLB_ERR_CAPACITY: c_int = 4;
    pub const XLB_ERR_ITER_LIMIT: c_int = 5;
    pub const XLB_ERR_CUDA: c_int = 6;
    pub const XLB_ERR_NCCL: c_int = 7;
    pub const XLB_ERR_TIMEOUT: c_int = 8;
    pub const XLB_ERR_UNSUPPORTED: c_int = 9;
    pub const XLB_ERR_NOT_FOUND: c_int = 10;

    // xlb_type: the reference's kernel type codes (crates/xlog-core/src/types.rs:33-62)
    pub const XLB_U32: u8 = 0;
    pub const XLB_U64: u8 = 1;
    pub const XLB_I32: u8 = 2;
    pub const XLB_I64: u8 = 3;
    pub const XLB_F32: u8 = 4;
    pub const XLB_F64: u8 = 5;
    pub const XLB_BOOL: u8 = 6;
    pub const XLB_SYMBOL: u8 = 7;

    pub const XLB_FLAG_PROFILE: u32 = 1;
    pub const XLB_FLAG_NO_DENSE: u32 = 2;
    pub const XLB_FLAG_KEEP_DELTAS: u32 = 4;
    pub const XLB_FLAG_SHUFFLE_ONLY: u32 = 8;
    pub const XLB_FLAG_NO_TUPLE_SET: u32 = 16;
    pub const XLB_FLAG_GENERAL_ONLY: u32 = 32;

    pub const XLB_JOIN_INNER: c_int = 0;
    pub const XLB_JOIN_SEMI: c_int = 1;
    pub const XLB_JOIN_ANTI: c_int = 2;

    pub const XLB_NODE_SCAN: u32 = 1;
    pub const XLB_NODE_FILTER: u32 = 2;
    pub const XLB_NODE_PROJECT: u32 = 3;
    pub const XLB_NODE_JOIN: u32 = 4;
    pub const XLB_NODE_UNION: u32 = 5;
    pub const XLB_NODE_DIFF: u32 = 6;
    pub const XLB_NODE_DISTINCT: u32 = 7;

    #[repr(C)]
    pub struct xlb_ctx {
        _private: [u8; 0],
    }
    #[repr(C)]
    pub struct xlb_rel {
        _private: [u8; 0],
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct xlb_schema {
        pub arity: u32,
        pub types: [u8; XLB_MAX_ARITY],
    }

    #[repr(C)]
    #[derive(Clone, Copy, Default)]
    pub struct xlb_config {
        pub device: i32,
        pub memory_budget_bytes: u64,
        pub max_iterations: u64,
        pub join_chunk_tuples: u64,
        pub flags: u32,
    }

    #[repr(C)]
    pub struct xlb_node {
        pub kind: u32,
        pub rel_id: u32,
        pub input: *const xlb_node,
        pub left: *const xlb_node,
        pub right: *const xlb_node,
        pub n_keys: u32,
        pub left_keys: [u32; XLB_MAX_KEYS],
        pub right_keys: [u32; XLB_MAX_KEYS],
        pub n_cols: u32,
        pub cols: [u32; XLB_MAX_ARITY],
        pub cmp: u32,
        pub cmp_lhs_col: u32,
        pub cmp_rhs_is_const: u32,
        pub cmp_rhs: u64,
        pub inputs: *const *const xlb_node,
        pub n_inputs: u32,
        pub join_type: u32,
    }

    #[repr(C)]
    pub struct xlb_rule {
        pub head: *const c_char,
        pub body: *const xlb_node,
        pub head_schema: xlb_schema,
    }

    #[repr(C)]
    pub struct xlb_scc {
        pub id: u32,
        pub is_recursive: u32,
        pub rules: *const xlb_rule,
        pub n_rules: u32,
    }

    #[repr(C)]
    pub struct xlb_plan {
        pub sccs: *const xlb_scc,
        pub n_sccs: u32,
    }

    /// ExecutionStats subset (crates/xlog-runtime/src/profiler.rs:172-233) + data-plane counters.
    #[repr(C)]
    #[derive(Clone, Copy, Default, Debug)]
    pub struct xlb_run_stats {
        pub iterations: u64,
        pub derived_tuples: u64,
        pub candidate_tuples: u64,
        pub kernel_launches: u64,
        pub peak_bytes: u64,
        pub ms_total: f64,
        pub ms_join: f64,
        pub ms_sort: f64,
        pub ms_setops: f64,
        pub ms_exchange: f64,
        pub exchange_bytes: u64,
        pub host_syncs: u64,
        pub ms_host_wait: f64,
        pub ms_host_total: f64,
        pub ms_host_alloc: f64,
    }

    #[repr(C)]
    #[derive(Clone, Copy)]
    pub struct xlb_kernel_profile {
        pub name: [c_char; 32],
        pub launches: u64,
        pub bytes: u64,
        pub ms: f64,
    }

    #[link(name = "xlb")]
    extern "C" {
        pub fn xlb_ctx_create(cfg: *const xlb_config, out: *mut *mut xlb_ctx) -> c_int;
        pub fn xlb_ctx_destroy(ctx: *mut xlb_ctx);
        pub fn xlb_last_error(ctx: *const xlb_ctx) -> *const c_char;
        pub fn xlb_memory_stats(ctx: *const xlb_ctx, allocated: *mut u64, peak: *mut u64) -> c_int;

        pub fn xlb_rel_from_host(ctx: *mut xlb_ctx, schema: *const xlb_schema, cols: *const *const c_void, rows: u64, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_rel_empty(ctx: *mut xlb_ctx, schema: *const xlb_schema, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_rel_rows(rel: *const xlb_rel, rows: *mut u64) -> c_int;
        pub fn xlb_rel_schema(rel: *const xlb_rel, schema: *mut xlb_schema) -> c_int;
        pub fn xlb_rel_is_canonical(rel: *const xlb_rel, canonical: *mut c_int) -> c_int;
        pub fn xlb_rel_to_host(ctx: *mut xlb_ctx, rel: *const xlb_rel, cols: *const *mut c_void, cap_rows: u64, rows: *mut u64) -> c_int;
        pub fn xlb_rel_clone(ctx: *mut xlb_ctx, rel: *const xlb_rel, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_rel_free(rel: *mut xlb_rel);
        pub fn xlb_rel_checksum(ctx: *mut xlb_ctx, rel: *const xlb_rel, digest: *mut u64) -> c_int;

        pub fn xlb_hash_join(ctx: *mut xlb_ctx, left: *const xlb_rel, right: *const xlb_rel, left_keys: *const u32, right_keys: *const u32,
                             n_keys: u32, join_type: c_int, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_sort(ctx: *mut xlb_ctx, rel: *const xlb_rel, key_cols: *const u32, n_keys: u32, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_dedup(ctx: *mut xlb_ctx, rel: *const xlb_rel, key_cols: *const u32, n_keys: u32, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_union(ctx: *mut xlb_ctx, ins: *const *const xlb_rel, n: u32, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_diff(ctx: *mut xlb_ctx, a: *const xlb_rel, b: *const xlb_rel, out: *mut *mut xlb_rel) -> c_int;
        pub fn xlb_groupby(ctx: *mut xlb_ctx, rel: *const xlb_rel, key_cols: *const u32, n_keys: u32, agg_cols: *const u32, agg_ops: *const u32,
                           n_aggs: u32, out: *mut *mut xlb_rel) -> c_int;

        pub fn xlb_register_relation(ctx: *mut xlb_ctx, rel_id: u32, name: *const c_char) -> c_int;
        pub fn xlb_store_put(ctx: *mut xlb_ctx, name: *const c_char, rel: *mut xlb_rel) -> c_int;
        pub fn xlb_store_get(ctx: *mut xlb_ctx, name: *const c_char, rel: *mut *const xlb_rel) -> c_int;
        pub fn xlb_store_remove(ctx: *mut xlb_ctx, name: *const c_char) -> c_int;
        pub fn xlb_execute_plan(ctx: *mut xlb_ctx, plan: *const xlb_plan, stats: *mut xlb_run_stats) -> c_int;

        pub fn xlb_dedup_sorted_u64_static(d_sorted: *const u64, n: u64, d_unique: *mut u64, d_count: *mut u64, cuda_stream: *mut c_void) -> c_int;
        pub fn xlb_dedup_sorted_u64_static_max() -> u64;
        pub fn xlb_static_last_error() -> *const c_char;

        pub fn xlb_profile_enable(ctx: *mut xlb_ctx, kernel: *const c_char) -> c_int;
        pub fn xlb_profile_read(ctx: *mut xlb_ctx, out: *mut xlb_kernel_profile, cap: u32, n: *mut u32) -> c_int;

        pub fn xlb_comm_unique_id(id: *mut u8) -> c_int;
        pub fn xlb_comm_init(ctx: *mut xlb_ctx, id: *const u8, rank: u32, world: u32) -> c_int;
        pub fn xlb_owner_of(key: u64, world: u32) -> u32;
    }
}

/// Safe layer: owned relations and a context whose methods carry the names and argument order of
/// the `CudaKernelProvider` methods they replace (crates/xlog-cuda/src/provider/relational.rs) and of
/// `Executor::{register_relation, put_relation, execute_plan}` (crates/xlog-runtime/src/executor/mod.rs).
pub mod safe {
    use super::ffi::*;
    use std::ffi::{CStr, CString};
    use std::os::raw::c_void;
    use std::ptr;

    /// The error classes of `XlogError` (crates/xlog-core/src/error.rs:8-100) a status maps onto.
    #[derive(Debug)]
    pub enum XlbError {
        Execution(String),
        Kernel(String),
        ResourceExhausted(String),
    }
    pub type Result<T> = std::result::Result<T, XlbError>;

    /// Owns one `xlb_rel` (the reference's `CudaBuffer`); dropping it frees the device memory.
    pub struct Relation {
        raw: *mut xlb_rel,
    }
    impl Drop for Relation {
        fn drop(&mut self) {
            if !self.raw.is_null() {
                unsafe { xlb_rel_free(self.raw) }
            }
        }
    }
    impl Relation {
        pub fn num_rows(&self) -> u64 {
            let mut n = 0u64;
            unsafe { xlb_rel_rows(self.raw, &mut n) };
            n
        }
        pub fn schema(&self) -> xlb_schema {
            let mut s = xlb_schema::default();
            unsafe { xlb_rel_schema(self.raw, &mut s) };
            s
        }
    }

    /// One context on one GPU.  Not `Sync`: a context is used from one thread at a time, as the
    /// reference's runtime is (crates/xlog-runtime/src/relation.rs:20-23).
    pub struct Context {
        raw: *mut xlb_ctx,
    }
    impl Drop for Context {
        fn drop(&mut self) {
            unsafe { xlb_ctx_destroy(self.raw) }
        }
    }

    impl Context {
        pub fn new(cfg: xlb_config) -> Result<Self> {
            let mut raw = ptr::null_mut();
            let st = unsafe { xlb_ctx_create(&cfg, &mut raw) };
            if st != XLB_OK {
                let msg = unsafe { CStr::from_ptr(xlb_last_error(ptr::null())) }.to_string_lossy().into_owned();
                return Err(classify(st, msg));
            }
            Ok(Context { raw })
        }

        fn check(&self, st: i32) -> Result<()> {
            if st == XLB_OK {
                return Ok(());
            }
            let msg = unsafe { CStr::from_ptr(xlb_last_error(self.raw)) }.to_string_lossy().into_owned();
            Err(classify(st, msg))
        }

        fn take(&self, st: i32, out: *mut xlb_rel) -> Result<Relation> {
            self.check(st)?;
            Ok(Relation { raw: out })
        }

        /// `create_buffer_from_slices` (provider/io.rs:75): one byte slice per column.
        pub fn create_buffer_from_slices(&self, cols: &[&[u8]], schema: xlb_schema, rows: u64) -> Result<Relation> {
            let ptrs: Vec<*const c_void> = cols.iter().map(|c| c.as_ptr() as *const c_void).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_rel_from_host(self.raw, &schema, ptrs.as_ptr(), rows, &mut out) };
            self.take(st, out)
        }

        /// `download_column::<u32>` for every column (provider/transfer.rs:22).
        pub fn download_u32(&self, rel: &Relation) -> Result<Vec<Vec<u32>>> {
            let n = rel.num_rows() as usize;
            let arity = rel.schema().arity as usize;
            let mut cols: Vec<Vec<u32>> = (0..arity).map(|_| vec![0u32; n]).collect();
            let ptrs: Vec<*mut c_void> = cols.iter_mut().map(|c| c.as_mut_ptr() as *mut c_void).collect();
            let mut rows = 0u64;
            self.check(unsafe { xlb_rel_to_host(self.raw, rel.raw, ptrs.as_ptr(), n as u64, &mut rows) })?;
            Ok(cols)
        }

        /// `hash_join_v2` (relational.rs:2926).
        pub fn hash_join_v2(&self, left: &Relation, right: &Relation, left_keys: &[usize], right_keys: &[usize], join_type: i32) -> Result<Relation> {
            let lk: Vec<u32> = left_keys.iter().map(|&k| k as u32).collect();
            let rk: Vec<u32> = right_keys.iter().map(|&k| k as u32).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_hash_join(self.raw, left.raw, right.raw, lk.as_ptr(), rk.as_ptr(), lk.len() as u32, join_type, &mut out) };
            self.take(st, out)
        }

        /// `sort` (relational.rs:1881).
        pub fn sort(&self, input: &Relation, key_cols: &[usize]) -> Result<Relation> {
            let k: Vec<u32> = key_cols.iter().map(|&c| c as u32).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_sort(self.raw, input.raw, k.as_ptr(), k.len() as u32, &mut out) };
            self.take(st, out)
        }

        /// `dedup` (relational.rs:238); no key columns = the full-row form.
        pub fn dedup(&self, input: &Relation, key_cols: &[usize]) -> Result<Relation> {
            let k: Vec<u32> = key_cols.iter().map(|&c| c as u32).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_dedup(self.raw, input.raw, k.as_ptr(), k.len() as u32, &mut out) };
            self.take(st, out)
        }

        /// `union_many_gpu` (relational.rs:859).
        pub fn union_many_gpu(&self, inputs: &[&Relation]) -> Result<Relation> {
            let ins: Vec<*const xlb_rel> = inputs.iter().map(|r| r.raw as *const xlb_rel).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_union(self.raw, ins.as_ptr(), ins.len() as u32, &mut out) };
            self.take(st, out)
        }

        /// `diff_gpu` (relational.rs:1102).
        pub fn diff_gpu(&self, a: &Relation, b: &Relation) -> Result<Relation> {
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_diff(self.raw, a.raw, b.raw, &mut out) };
            self.take(st, out)
        }

        /// `groupby_multi_agg` (provider/groupby.rs:66): (value column, aggregation) pairs.
        pub fn groupby_multi_agg(&self, input: &Relation, key_cols: &[usize], aggs: &[(usize, u32)]) -> Result<Relation> {
            let k: Vec<u32> = key_cols.iter().map(|&c| c as u32).collect();
            let cols: Vec<u32> = aggs.iter().map(|a| a.0 as u32).collect();
            let ops: Vec<u32> = aggs.iter().map(|a| a.1).collect();
            let mut out = ptr::null_mut();
            let st = unsafe { xlb_groupby(self.raw, input.raw, k.as_ptr(), k.len() as u32, cols.as_ptr(), ops.as_ptr(), ops.len() as u32, &mut out) };
            self.take(st, out)
        }

        /// `Executor::register_relation` (executor/mod.rs:1242).
        pub fn register_relation(&self, rel_id: u32, name: &str) -> Result<()> {
            let n = CString::new(name).map_err(|e| XlbError::Execution(e.to_string()))?;
            self.check(unsafe { xlb_register_relation(self.raw, rel_id, n.as_ptr()) })
        }

        /// `Executor::put_relation` (executor/mod.rs:587): the store takes ownership.
        pub fn put_relation(&self, name: &str, mut rel: Relation) -> Result<()> {
            let n = CString::new(name).map_err(|e| XlbError::Execution(e.to_string()))?;
            let raw = std::mem::replace(&mut rel.raw, ptr::null_mut());
            let st = unsafe { xlb_store_put(self.raw, n.as_ptr(), raw) };
            if st != XLB_OK {
                rel.raw = raw; // not taken: freed when `rel` drops
            }
            self.check(st)
        }

        /// `Executor::execute_plan` (executor/mod.rs:1404-1469) on a plan lowered to `xlb_plan`.
        ///
        /// # Safety
        /// Every pointer reachable from `plan` must stay valid for the duration of the call.
        pub unsafe fn execute_plan(&self, plan: &xlb_plan) -> Result<xlb_run_stats> {
            let mut stats = xlb_run_stats::default();
            self.check(xlb_execute_plan(self.raw, plan, &mut stats))?;
            Ok(stats)
        }

        /// `store().get(name)` (executor/mod.rs:562) followed by a download of u32 columns.
        pub fn get_u32(&self, name: &str) -> Result<Vec<Vec<u32>>> {
            let n = CString::new(name).map_err(|e| XlbError::Execution(e.to_string()))?;
            let mut borrowed: *const xlb_rel = ptr::null();
            self.check(unsafe { xlb_store_get(self.raw, n.as_ptr(), &mut borrowed) })?;
            let view = Relation { raw: borrowed as *mut xlb_rel };
            let cols = self.download_u32(&view);
            std::mem::forget(view); // borrowed from the store: not ours to free
            cols
        }
    }

    fn classify(st: i32, msg: String) -> XlbError {
        match st {
            XLB_ERR_RESOURCE_EXHAUSTED => XlbError::ResourceExhausted(msg),
            XLB_ERR_INVALID | XLB_ERR_ITER_LIMIT | XLB_ERR_UNSUPPORTED | XLB_ERR_NOT_FOUND => XlbError::Execution(msg),
            _ => XlbError::Kernel(msg), // TYPE, CAPACITY, CUDA, NCCL, TIMEOUT
        }
    }
}
