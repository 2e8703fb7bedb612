// NOT COMPILED in this repository's build image (no Rust toolchain); see ../README.md.
//
// Additions to helium/src/cuda/instr.rs (enum Instr, :20-99) and helium/src/cuda.rs (make_instr_for_op,
// :33-60).  Graph recording, autodiff, plan generation, allocation, streams and events stay as they are;
// only the bodies of precompile / execute / can_fuse_with change, plus one new variant for matmuls.

use helium_b200_sys as sys;
use std::os::raw::c_void;
use std::sync::Arc;

pub enum Instr {
    PointwiseGraph(PointwiseGraph),
    PermuteDims(PermuteDims),
    FusedMatmul(FusedMatmul), // new: Op::Matmul (cuda.rs:55-58 builds it instead of CudnnGraph)
    Conv2d(Conv2d),           // new: Op::Conv / ConvBackwardData / ConvBackwardFilter through he_plan_conv2d (see below)
}

pub struct FusedMatmul {
    subgraph: OpSubgraph,
    input_order: Vec<NodeId>,
    leaf_order: Vec<NodeId>,
}

struct PlanHandle(*mut sys::he_plan);
unsafe impl Send for PlanHandle {}
unsafe impl Sync for PlanHandle {} // plans are immutable after creation
impl Drop for PlanHandle {
    fn drop(&mut self) {
        unsafe { sys::he_plan_destroy(self.0) }
    }
}

#[derive(Copy, Clone)]
enum PlanKind {
    Pointwise,
    Matmul,
}

/// OpSubgraph -> he_graph_desc records.  Subgraph inputs come first (HE_OP_INPUT records carry only the
/// descriptor), then the nodes in NodeId order (`OpSubgraph::nodes()` is sorted,
/// helium-ir/src/opgraph/subgraph.rs:40), each operand rewritten to its index in the flat list.
fn flatten(sub: &OpSubgraph) -> (Vec<sys::he_node>, Vec<i32>, Vec<NodeId>, Vec<NodeId>) {
    let mut index = AHashMap::new();
    let mut nodes = Vec::new();
    let inputs: Vec<NodeId> = sub.inputs().collect();
    for id in &inputs {
        index.insert(*id, nodes.len() as i32);
        nodes.push(input_record(sub.graph().get(*id).descriptor()));
    }
    for id in sub.nodes() {
        let Node::Intermediate(Intermediate { op, descriptor }) = sub.graph().get(id) else { unreachable!() };
        let mut n = record_for(op, descriptor);
        for (k, src) in op.inputs().iter().enumerate() {
            n.r#in[k] = index[src];
        }
        index.insert(id, nodes.len() as i32);
        nodes.push(n);
    }
    let leafs: Vec<NodeId> = sub.leafs().collect();
    let outputs = leafs.iter().map(|l| index[l]).collect();
    (nodes, outputs, inputs, leafs)
}

fn blank(kind: i32, d: &Descriptor) -> sys::he_node {
    let mut shape = [0i64; sys::HE_MAX_RANK];
    for (k, dim) in d.shape.dims().iter().enumerate() {
        shape[k] = *dim as i64;
    }
    sys::he_node { kind, sub_op: 0, r#in: [-1; 3], dtype: d.data_type as i32, rank: d.shape.num_dims() as i32,
                   shape, const_bits: 0, axis_a: 0, axis_b: 0, axes: 0 }
}

fn input_record(d: &Descriptor) -> sys::he_node {
    blank(sys::HE_OP_INPUT, d)
}

/// One record per `Op` variant (helium-ir/src/opgraph/op.rs:15-30).  The enum orders of UnaryPointwiseOp
/// (:291-304), BinaryPointwiseOp (:315-328), CompareOp and ReduceOp are the orders of he_unary_op,
/// he_binary_op, he_compare_op and he_reduce_op.
fn record_for(op: &Op, d: &Descriptor) -> sys::he_node {
    match op {
        Op::Constant(c) => { let mut n = blank(sys::HE_OP_CONSTANT, d); n.const_bits = c.value.to_bits(); n }
        Op::UnaryPointwise(u) => { let mut n = blank(sys::HE_OP_UNARY, d); n.sub_op = u.op as i32; n }
        Op::BinaryPointwise(b) => { let mut n = blank(sys::HE_OP_BINARY, d); n.sub_op = b.op as i32; n }
        Op::ChangeDataType(_) => blank(sys::HE_OP_CAST, d),
        Op::Reduce(r) => {
            let mut n = blank(sys::HE_OP_REDUCE, d);
            let in_rank = d.shape.num_dims() as u32 - 1 + r.depth; // [.., 1] replaces the last `depth` dims
            n.sub_op = r.op as i32;
            n.axes = ((1u32 << r.depth) - 1) << (in_rank - r.depth);
            n
        }
        Op::Broadcast(_) => blank(sys::HE_OP_BROADCAST, d), // only the output shape is needed
        Op::Reshape(_) => blank(sys::HE_OP_RESHAPE, d),
        Op::SwapDims(s) => { let mut n = blank(sys::HE_OP_SWAP_DIMS, d); n.axis_a = s.axis_a as i32; n.axis_b = s.axis_b as i32; n }
        Op::Compare(c) => { let mut n = blank(sys::HE_OP_COMPARE, d); n.sub_op = c.op as i32; n }
        Op::Select(_) => blank(sys::HE_OP_SELECT, d), // in = {lhs, rhs, selector}
        Op::Matmul(m) => { let mut n = blank(sys::HE_OP_MATMUL, d); n.sub_op = precision_code(m.precision); n }
        _ => unreachable!("op is not served by helium_b200"),
    }
}

fn precision_code(p: Precision) -> i32 {
    match p {
        Precision::MulF32AccumF32 => sys::HE_PREC_F32_F32,
        Precision::MulTf32AccumF32 => sys::HE_PREC_TF32_F32,
        Precision::MulBf16AccumF32 => sys::HE_PREC_BF16_F32,
        Precision::MulF16AccumF32 => sys::HE_PREC_F16_F32,
        Precision::MulF16AccumF16 => sys::HE_PREC_F16_F16,
        Precision::MulF8AccumF32 { mode_a, mode_b } => sys::he_prec_f8(sys::HE_PREC_F8_F32, mode_a as i32, mode_b as i32),
        Precision::MulF8AccumF16 { mode_a, mode_b } => sys::he_prec_f8(sys::HE_PREC_F8_F16, mode_a as i32, mode_b as i32),
    }
}

// precompile: was NVRTC + cuModuleLoadData (pointwise.rs:40-54, permute_dims.rs:55-83)
fn plan_for(sub: &OpSubgraph, cx: &CudaContext, kind: PlanKind) -> Arc<PlanHandle> {
    static CACHE: Cache<OpSubgraph, Arc<PlanHandle>> = Cache::with_capacity(1024); // same key as today's kernel cache
    CACHE.get_or_insert(sub, || {
        let (nodes, outputs, ..) = flatten(sub);
        let desc = sys::he_graph_desc { num_nodes: nodes.len() as i32, nodes: nodes.as_ptr(),
                                        num_outputs: outputs.len() as i32, outputs: outputs.as_ptr() };
        let mut plan = std::ptr::null_mut();
        let st = unsafe {
            match kind {
                PlanKind::Pointwise => sys::he_plan_pointwise(cx.he_ctx(), &desc, &mut plan),
                PlanKind::Matmul => sys::he_plan_fused_matmul(cx.he_ctx(), &desc, &mut plan),
            }
        };
        assert_eq!(st, sys::HE_OK, "{}", sys::last_error()); // the reference panics on failure (pointwise.rs:50-51)
        Arc::new(PlanHandle(plan))
    })
}

impl FusedMatmul {
    pub fn precompile(&self, cx: &CudaContext) {
        plan_for(&self.subgraph, cx, PlanKind::Matmul);
    }

    // execute: was cudnnBackendExecute (cudnn_graph.rs:64-105)
    pub fn execute(&self, tensors: &TensorMap<Cuda>, stream: &CudaStream, cx: &CudaContext,
                   hold_allocations: &mut Vec<DeviceMemory>, allocation_stream: AllocationStreamId) {
        let plan = plan_for(&self.subgraph, cx, PlanKind::Matmul);
        let ins: Vec<*const c_void> = self.input_order.iter().map(|n| tensors.get_storage(*n).device_ptr() as _).collect();
        let outs: Vec<*mut c_void> = self.leaf_order.iter().map(|n| tensors.get_storage(*n).device_ptr() as _).collect();
        let mut ws_bytes = 0usize;
        unsafe { sys::he_plan_workspace_bytes(plan.0, &mut ws_bytes) };
        let ws = (ws_bytes > 0).then(|| cx.allocator().allocate_in_stream(ws_bytes as u64, 256, allocation_stream));
        let st = unsafe {
            sys::he_launch(plan.0, ins.as_ptr(), outs.as_ptr(),
                           ws.as_ref().map_or(std::ptr::null_mut(), |m| m.device_ptr() as _), stream.raw() as _)
        };
        assert_eq!(st, sys::HE_OK, "{}", sys::last_error());
        hold_allocations.extend(ws); // alive until the step ends, like the cuDNN workspace (cudnn_graph.rs:75-92)
    }
}

impl Instruction<Cuda> for Instr {
    fn can_fuse_with(&self, next: &Self, _g: &Arc<OpGraph>) -> bool {
        let kind = match (self, next) {
            (Instr::PointwiseGraph(_), Instr::PointwiseGraph(_)) => 0,
            (Instr::PermuteDims(_), Instr::PermuteDims(_)) => 1,
            // pointwise prologues fold into the mainloop, pointwise / reduction successors into the epilogue
            (Instr::FusedMatmul(_), Instr::PointwiseGraph(_)) | (Instr::PointwiseGraph(_), Instr::FusedMatmul(_)) => 2,
            // swap_dims of the last two dims in front of a matmul becomes an operand-major flag
            (Instr::PermuteDims(_), Instr::FusedMatmul(_)) => 2,
            // swap_dims -> reduce is read through the swapped view by the reduction kernel
            (Instr::PermuteDims(_), Instr::PointwiseGraph(_)) => 0,
            _ => return false,
        };
        let merged = self.subgraph().merge_with(next.subgraph());
        let (nodes, outputs, ..) = flatten(&merged);
        let desc = sys::he_graph_desc { num_nodes: nodes.len() as i32, nodes: nodes.as_ptr(),
                                        num_outputs: outputs.len() as i32, outputs: outputs.as_ptr() };
        // 2 = hand-written kernel, 1 = interpreter tier, 0 = cannot run as one kernel
        unsafe { sys::he_plan_supported(CudaContext::current().he_ctx(), &desc, kind) > 0 }
    }
}

/// Convolutions do not travel as graph records: one plan per (kind, Conv2dParams, image size, fusion).
pub struct Conv2d {
    kind: i32, // sys::HE_CONV_FWD / HE_CONV_BWD_DATA / HE_CONV_BWD_FILTER
    params: sys::he_conv2d_params,
    fusion: sys::he_conv2d_fusion,
    batch: i32,
    in_h: i32,
    in_w: i32,
    dtype: i32,
    input_order: Vec<NodeId>, // operand order of include/helium_b200.h for `kind`
    leaf_order: Vec<NodeId>,
}

fn conv_params(p: &Conv2dParams) -> sys::he_conv2d_params {
    sys::he_conv2d_params {
        in_channels: p.in_channels as i32, out_channels: p.out_channels as i32,
        kernel_h: p.kernel_size[0] as i32, kernel_w: p.kernel_size[1] as i32,
        stride_h: p.stride[0] as i32, stride_w: p.stride[1] as i32,
        dilation_h: p.dilation[0] as i32, dilation_w: p.dilation[1] as i32,
        padding_mode: match p.padding_mode { PaddingMode::Same => 0, PaddingMode::Valid => 1, PaddingMode::Full => 2 },
    }
}

impl Conv2d {
    fn plan(&self, cx: &CudaContext) -> *mut sys::he_plan {
        let mut plan = std::ptr::null_mut();
        let st = unsafe {
            sys::he_plan_conv2d(cx.he_ctx(), self.kind, &self.params, self.batch, self.in_h, self.in_w, self.dtype, &self.fusion, &mut plan)
        };
        assert_eq!(st, sys::HE_OK, "{}", sys::last_error());
        plan // cached per Conv2d like the plans above; launched exactly like FusedMatmul::execute
    }
}

/// Data-parallel step: one call per gradient bucket, as soon as the instruction that produces the bucket has
/// been enqueued on `stream`; `finish` before the optimiser instruction.  Mean, not sum, because
/// `cross_entropy_loss` divides by the local batch (helium/src/loss.rs:5-8).
pub struct GradExchange {
    comm: *mut sys::he_comm,
    comm_stream: CudaStream,
}

impl GradExchange {
    pub fn reduce_bucket(&self, stream: &CudaStream, bucket: &[(*mut c_void, usize)], dtype: i32) {
        let ev = stream.record_event();
        self.comm_stream.wait(&ev);
        let bufs: Vec<*mut c_void> = bucket.iter().map(|b| b.0).collect();
        let counts: Vec<usize> = bucket.iter().map(|b| b.1).collect();
        let st = unsafe {
            sys::he_allreduce_grads(self.comm, bufs.as_ptr(), counts.as_ptr(), bufs.len() as i32, dtype, 1,
                                    self.comm_stream.raw() as _)
        };
        assert_eq!(st, sys::HE_OK, "{}", sys::last_error());
    }

    pub fn finish(&self, stream: &CudaStream) {
        stream.wait(&self.comm_stream.record_event());
        assert_eq!(unsafe { sys::he_comm_poll(self.comm) }, sys::HE_OK, "{}", sys::last_error());
    }
}
