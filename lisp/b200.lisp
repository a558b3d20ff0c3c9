;;;; BACKEND=B200 for Caten: one new backend behind the BYOC interface, over libcaten_b200.so.
;;;;
;;;; Where this file goes: source/byoc/b200.lisp of hikettei/Caten, listed in source/byoc/caten.byoc.asd
;;;; next to metal.lisp.  Everything else of Caten stays as it is: `caten`, `forward`, `proceed` and the
;;;; external/llm GPT-2 graph run unchanged with (ctx:with-contextvar (:BACKEND "B200") ...).
;;;;
;;;; What it supplies (the contract of source/codegen/backend.lisp:22-34; template source/byoc/metal.lisp):
;;;;   B200Buffer          device memory: the six generics of source/runtime/buffer.lisp:78-89
;;;;   B200Runtime         a GraphRuntime that (i) uploads LispBuffer weights when an :Allocate node
;;;;                       names them (source/runtime/runtime.lisp:228-243) and (ii) collapses the
;;;;                       :JIT_KERNEL run of the GPT-2 Transformer into one caten_b200_gpt2_step call
;;;;   B200-Renderer       %render-kernel / %compile-kernel that match each Schedule-Item by the
;;;;                       :_lowering_history of its nodes (source/api/iseq.lisp:359-361) and return a
;;;;                       lambda form calling the matching C entry point; no C is generated and an
;;;;                       item that matches nothing is an error at compile time (no CPU fallback)
;;;;   B200-Auto-Scheduler an auto-scheduler configuration that asks for nothing (ISL is not used)
;;;;   loader patch        external/gguf: tensors stay in their GGUF block form, :Q4_0 added
;;;;   make-gpt2 :batch    the batched variant of apps/gpt2/gpt2.lisp:82-93
;;;;   dist-*              batch sharding over the GPUs of one box through caten_b200_dist_*
;;;;
;;;; Every foreign name and argument list below is checked against include/caten_b200.h by
;;;; tests/test_lisp_binding.py.  The file has not been executed: no Common Lisp implementation exists
;;;; on the machines this backend is built and measured on.

(defpackage :caten/byoc/b200
  (:use
   :cl :caten/air :caten/codegen/expr :caten/codegen/renderer :caten/codegen/shape-inference
   :caten/runtime/buffer :caten/runtime/runtime :caten/codegen/helpers :caten/codegen/blueprint
   :caten/common.dtype :caten/codegen/backend :cffi)
  (:import-from :caten/codegen/config #:define-auto-scheduler)
  (:export
   #:B200Buffer #:B200Runtime #:B200-Renderer #:B200-Auto-Scheduler
   #:*precision* #:upload-packed-weight #:make-gpt2-b200 #:b200-gpt2-forward
   #:dist-init #:dist-shard #:dist-bcast-weights #:dist-gather-ids))

(in-package :caten/byoc/b200)

;;; ~~ library, context, errors ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(define-foreign-library libcaten-b200
  (t (:default "libcaten_b200")))

(defvar *library-loaded* nil)
(defvar *ctx* (null-pointer) "The caten_b200_ctx of this Lisp image (one device, one stream).")
(defvar *device* 0 "CUDA device ordinal; under a multi-process launch, the local rank.")

;; status codes and enums of include/caten_b200.h
(defconstant +ok+ 0)
(defconstant +act-none+ 0) (defconstant +act-gelu+ 1) (defconstant +act-relu+ 2)
(defconstant +prec-fp32+ 0) (defconstant +prec-bf16+ 1) (defconstant +prec-bf16x3+ 2)
(defconstant +dist-id-bytes+ 128)

(defparameter *precision* +prec-bf16x3+
  "Arithmetic of the Linear kernels when more than four rows are multiplied at once:
+prec-fp32+ (CUDA cores, bit-identical to the C the CLANG backend renders), +prec-bf16+, +prec-bf16x3+.")

(defun ggml-type-id (keyword)
  "ggml type keyword (external/gguf/tensor-info.lisp:3-34) -> the id the C library takes."
  (ecase keyword
    (:F32 0) (:F16 1) (:Q4_0 2) (:Q4_1 3) (:Q5_0 6) (:Q5_1 7) (:Q8_0 8)
    (:Q2_K 10) (:Q3_K 11) (:Q4_K 12) (:Q5_K 13) (:Q6_K 14)))

(defun check (rc)
  "Every entry point returns an int status; non-zero becomes a Lisp error carrying the library's message
(the way a failing gcc surfaces in source/byoc/clang.lisp:150-156)."
  (unless (= rc +ok+)
    (error "caten_b200 (status ~a): ~a" rc
           (foreign-funcall "caten_b200_last_error" :pointer *ctx* :string)))
  rc)

(defun ensure-ctx ()
  (unless *library-loaded*
    (use-foreign-library libcaten-b200)
    (setf *library-loaded* t))
  (when (null-pointer-p *ctx*)
    (with-foreign-object (p :pointer)
      (let ((rc (foreign-funcall "caten_b200_init" :int *device* :pointer p :int)))
        (unless (= rc +ok+)
          (error "caten_b200_init (status ~a): ~a" rc
                 (foreign-funcall "caten_b200_last_error" :pointer (null-pointer) :string))))
      (setf *ctx* (mem-ref p :pointer))))
  *ctx*)

(defun b200-sync () (check (foreign-funcall "caten_b200_sync" :pointer (ensure-ctx) :int)))

(defun b200-shutdown ()
  (unless (null-pointer-p *ctx*)
    (check (foreign-funcall "caten_b200_destroy" :pointer *ctx* :int))
    (setf *ctx* (null-pointer))))

;;; ~~ buffers (source/runtime/buffer.lisp:78-89) ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(defclass B200Buffer (AbstractBuffer)
  ((weight :initform nil :accessor b200-buffer-weight
           :documentation "caten_b200_weight handle when the buffer holds a Linear weight in GGUF block form; then
buffer-dtype still says what the graph believes (:float32) and the kernels consult this slot.")
   (ggml-type :initform nil :accessor b200-buffer-ggml-type))
  (:documentation "buffer-value is a device pointer (rank > 0) or an immediate Lisp number (rank 0), as MetalBuffer does
(source/byoc/metal.lisp:112-121)."))

(defun buffer-nbytes (buffer)
  (* (buffer-storage-size buffer) (dtype/size-of (buffer-dtype buffer))))

(defmethod open-buffer ((runtime GraphRuntime) (buffer B200Buffer))
  ;; "Fills the (buffer-value buffer) with zero": caten_b200_malloc returns zero-filled memory
  (if (= 0 (buffer-nrank buffer))
      (setf (buffer-value buffer)
            (if (eql (buffer-dtype buffer) :bool) nil (coerce 0 (dtype->lisp (buffer-dtype buffer)))))
      (with-foreign-object (p :pointer)
        (check (foreign-funcall "caten_b200_malloc" :pointer (ensure-ctx) :size (buffer-nbytes buffer) :pointer p :int))
        (setf (buffer-value buffer) (mem-ref p :pointer)))))

(defmethod close-buffer ((runtime GraphRuntime) (buffer B200Buffer))
  (when (b200-buffer-weight buffer)
    (check (foreign-funcall "caten_b200_weight_free" :pointer *ctx* :pointer (b200-buffer-weight buffer) :int))
    (setf (b200-buffer-weight buffer) nil))
  (when (pointerp (buffer-value buffer))
    (check (foreign-funcall "caten_b200_free" :pointer *ctx* :pointer (buffer-value buffer) :int))
    (setf (buffer-value buffer) nil)))

(defmethod transfer-from-array ((runtime GraphRuntime) (buffer B200Buffer) array)
  ;; host -> device; `array` is a specialised simple-array whose element type matches the dtype
  (if (= 0 (buffer-nrank buffer))
      (setf (buffer-value buffer) (if (arrayp array) (aref array 0) array))
      (with-pointer-to-vector-data (src array)
        (check (foreign-funcall "caten_b200_h2d" :pointer *ctx* :pointer (buffer-value buffer) :pointer src
                                :size (buffer-nbytes buffer) :int)))))

(defmethod transfer-into-array ((buffer B200Buffer))
  ;; device -> host, synchronising
  (when (or (numberp (buffer-value buffer)) (typep (buffer-value buffer) 'boolean))
    (return-from transfer-into-array (buffer-value buffer)))
  (let ((out (make-array (buffer-storage-size buffer) :element-type (dtype->lisp (buffer-dtype buffer)))))
    (with-pointer-to-vector-data (dst out)
      (check (foreign-funcall "caten_b200_d2h" :pointer *ctx* :pointer dst :pointer (buffer-value buffer)
                              :size (buffer-nbytes buffer) :int)))
    out))

(defmethod copy-buffer-value ((runtime GraphRuntime) (buffer B200Buffer))
  ;; "Returns a copy of the buffer value" (forward copies every output, source/api/iseq.lisp:524-527)
  (if (pointerp (buffer-value buffer))
      (with-foreign-object (p :pointer)
        (check (foreign-funcall "caten_b200_malloc" :pointer *ctx* :size (buffer-nbytes buffer) :pointer p :int))
        (check (foreign-funcall "caten_b200_d2d" :pointer *ctx* :pointer (mem-ref p :pointer)
                                :pointer (buffer-value buffer) :size (buffer-nbytes buffer) :int))
        (mem-ref p :pointer))
      (buffer-value buffer)))

(defmethod bref ((buffer B200Buffer) idx)
  ;; one element for printing (pprint-buffer): a small synchronous device -> host copy
  (if (pointerp (buffer-value buffer))
      (let ((cffi-type (->cffi-dtype (buffer-dtype buffer)))
            (size (dtype/size-of (buffer-dtype buffer))))
        (with-foreign-object (one cffi-type)
          (check (foreign-funcall "caten_b200_d2h" :pointer *ctx* :pointer one
                                  :pointer (inc-pointer (buffer-value buffer) (* idx size)) :size size :int))
          (mem-ref one cffi-type)))
      (buffer-value buffer)))

;;; ~~ weights kept in GGUF block form (external/gguf/tensor-info.lisp:104-120) ~~~~~~~~~~~~~~~~~~~~~~~~~

(defun upload-packed-weight (ggml-type raw-bytes rows cols)
  "raw-bytes: the (unsigned-byte 8) vector of the tensor as it sits in the file.  Returns a B200Buffer of
logical shape (rows cols) that carries the device weight handle; nothing is dequantised."
  (declare (type keyword ggml-type) (type (simple-array (unsigned-byte 8) (*)) raw-bytes))
  (ensure-ctx)
  (let ((expected (foreign-funcall "caten_b200_weight_nbytes" :int (ggml-type-id ggml-type) :int64 rows :int64 cols :int64)))
    (assert (= expected (length raw-bytes)) ()
            "upload-packed-weight: a ~a tensor of ~ax~a takes ~a bytes, got ~a" ggml-type rows cols expected (length raw-bytes)))
  (let ((buffer (make-buffer (list rows cols) (list cols 1) :float32 nil :device 'B200Buffer)))
    (with-foreign-object (w :pointer)
      (with-pointer-to-vector-data (src raw-bytes)
        (check (foreign-funcall "caten_b200_weight_upload" :pointer *ctx* :int (ggml-type-id ggml-type) :pointer src
                                :int64 rows :int64 cols :pointer w :int)))
      (setf (b200-buffer-weight buffer) (mem-ref w :pointer)
            (b200-buffer-ggml-type buffer) ggml-type
            ;; never dereferenced as fp32: kernels that meet this buffer use the handle
            (buffer-value buffer) (mem-ref w :pointer)))
    buffer))

(defun weight-handle (buffer)
  "The caten_b200_weight of a buffer used as a Linear weight.  A plain fp32 device buffer (a weight that came
through the fp32 path, e.g. random initialisation) is wrapped once, from device memory."
  (or (b200-buffer-weight buffer)
      (destructuring-bind (rows cols) (last (buffer-shape buffer) 2)
        (with-foreign-object (w :pointer)
          (check (foreign-funcall "caten_b200_weight_upload_device" :pointer *ctx* :int (ggml-type-id :F32)
                                  :pointer (buffer-value buffer) :int64 rows :int64 cols :pointer w :int))
          (setf (b200-buffer-ggml-type buffer) :F32
                (b200-buffer-weight buffer) (mem-ref w :pointer))))))

(defun dequantize-on-device (buffer)
  "fp32 values of a packed weight: what `dequantize` (external/gguf/dequantize.lisp:8) returns, bit for bit."
  (destructuring-bind (rows cols) (buffer-shape buffer)
    (let ((out (make-array (* rows cols) :element-type 'single-float)))
      (with-foreign-object (p :pointer)
        (check (foreign-funcall "caten_b200_malloc" :pointer *ctx* :size (* 4 rows cols) :pointer p :int))
        (check (foreign-funcall "caten_b200_weight_dequant" :pointer *ctx* :pointer (weight-handle buffer)
                                :pointer (mem-ref p :pointer) :int))
        (with-pointer-to-vector-data (dst out)
          (check (foreign-funcall "caten_b200_d2h" :pointer *ctx* :pointer dst :pointer (mem-ref p :pointer)
                                  :size (* 4 rows cols) :int)))
        (check (foreign-funcall "caten_b200_free" :pointer *ctx* :pointer (mem-ref p :pointer) :int)))
      out)))

;; Loader patch.  external/gguf/tensor-info.lisp:71-77 calls (dequantize ggml-type stream tensor-info) and
;; tensor-info->tensor (:104-120) wraps the resulting single-float array in a LispBuffer.  Under BACKEND=B200
;; a 2-D tensor keeps its raw block bytes instead; :Q4_0, which the reference signals "Not ready" for
;; (tensor-info.lisp:41), is one of the formats the kernels consume packed.
(defstruct (Packed-Blocks (:constructor make-packed-blocks (ggml-type bytes rows cols)))
  ggml-type bytes rows cols)

(defun packed-type-p (ggml-type) (member ggml-type '(:Q4_0 :Q8_0 :F16 :Q4_1 :Q5_0 :Q5_1 :Q2_K :Q3_K :Q4_K :Q5_K :Q6_K)))

(defun read-packed-blocks (ggml-type aligned-buffer tensor-info)
  "Replacement body of `dequantize` for 2-D tensors when (ctx:getenv :BACKEND) is B200: reads the tensor's bytes
unchanged.  `aligned-buffer` is the fast-io input buffer positioned at the tensor (tensor-info.lisp:71-77)."
  (destructuring-bind (cols rows) (caten/gguf:tensor-info-dimensions tensor-info)  ; GGUF lists the contiguous dim first
    (let* ((n (foreign-funcall "caten_b200_weight_nbytes" :int (ggml-type-id ggml-type) :int64 rows :int64 cols :int64))
           (bytes (make-array n :element-type '(unsigned-byte 8))))
      (fast-io:fast-read-sequence bytes aligned-buffer)
      (make-packed-blocks ggml-type bytes rows cols))))

(defmethod caten/gguf:dequantize :around (type-id aligned-buffer tensor-info)
  (if (and (string-equal (princ-to-string (ctx:getenv :BACKEND)) "B200")
           (= 2 (caten/gguf:tensor-info-n-dimension tensor-info))
           (packed-type-p type-id))
      (read-packed-blocks type-id aligned-buffer tensor-info)
      (call-next-method)))

(defun packed-tensor-info->tensor (tensor-info)
  "`tensor-info->tensor` for a tensor read by read-packed-blocks: a :float32 tensor of the logical shape whose
buffer is a B200Buffer carrying the packed weight."
  (let* ((pb (caten/gguf:tensor-info-buffer tensor-info))
         (buffer (upload-packed-weight (packed-blocks-ggml-type pb) (packed-blocks-bytes pb)
                                       (packed-blocks-rows pb) (packed-blocks-cols pb)))
         (out (caten/api:make-tensor (list (packed-blocks-rows pb) (packed-blocks-cols pb)) :dtype :float32 :from buffer)))
    (setf (caten/api:tensor-buffer out) buffer)
    out))

;;; ~~ runtime ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(defclass B200Runtime (GraphRuntime)
  ((gpt2 :initform nil :accessor b200-runtime-gpt2
         :documentation "caten_b200_gpt2 handle once the :JIT_KERNEL run of the Transformer has been collapsed.")
   (gpt2-batch :initform 1 :accessor b200-runtime-gpt2-batch))
  (:documentation "Constructible with an empty graph and :renderer nil, as get-global-runtime does
(source/api/tensor.lisp:309-317).  Scalar VM ops stay in Lisp; kernels are asynchronous on the context's stream
and only transfer-into-array / bref / copy-buffer-value wait for the GPU."))

(defmethod initialize-instance :after ((runtime B200Runtime) &key)
  (ensure-ctx))

(defun ->b200-buffer (runtime buffer)
  "A LispBuffer (weights loaded by load-state-dict, inputs built by change-facet) moved to the device once."
  (if (or (typep buffer 'B200Buffer) (not (buffer-p buffer)) (not (arrayp (buffer-value buffer))))
      buffer
      (let ((dev (make-buffer (buffer-shape buffer) (buffer-stride buffer) (buffer-dtype buffer) (buffer-views buffer)
                              :device 'B200Buffer)))
        (open-buffer runtime dev)
        (transfer-from-array runtime dev (buffer-value buffer))
        dev)))

;; :Allocate with :from names a realised buffer (a parameter or an input): upload it on first sight and
;; keep the device copy in the node, so later forwards reuse it (source/runtime/runtime.lisp:228-243).
(defmethod realize-node :around ((node-type (eql :Allocate)) (runtime B200Runtime) node args)
  (let ((from (getattr node :from)))
    (cond
      ((or (null from) *supress-allocate-mode*) (call-next-method))
      ((symbolp from)
       (let ((val (runtime-getvar runtime from)))
         (assert (buffer-p val) () "The :from attribute in the ~a node should be a buffer or a symbol." node)
         (let ((dev (->b200-buffer runtime val)))
           (unless (eq dev val) (runtime-setvar runtime from dev))
           dev)))
      ((buffer-p from)
       (let ((dev (->b200-buffer runtime from)))
         (unless (eq dev from) (setf (getattr node :from) dev))
         dev))
      (t (error "The :from attribute in the ~a node should be a buffer or a symbol." node)))))

(defmethod runtime-invoke-jit-kernel ((runtime B200Runtime) kernel-info node args)
  ;; rank-0 arguments arrive as numbers, the rest as B200Buffers (source/codegen/runner.lisp:23-32)
  (apply (caten/codegen/jit:compiled-kernel-caller kernel-info) args))

(defmethod free-runtime :after ((runtime B200Runtime))
  (when (b200-runtime-gpt2 runtime)
    (check (foreign-funcall "caten_b200_gpt2_destroy" :pointer (b200-runtime-gpt2 runtime) :int))
    (setf (b200-runtime-gpt2 runtime) nil)))

;;; ~~ renderer: graph-pattern dispatch ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(defclass B200-Renderer (Renderer) ()
  (:documentation "Emits no source text.  %render-kernel classifies a Schedule-Item and returns a printable plan;
%compile-kernel turns the plan into the lambda form stored in :compiled-object (compiled by
source/codegen/jit.lisp:118-120)."))

(defmethod get-default-renderer ((id (eql :b200))) (make-instance 'B200-Renderer))

(define-auto-scheduler (B200-Auto-Scheduler ()) :n-global-loop 0
  :documentation "Nothing to schedule: the kernels are hand-written.  Run with AUTO_SCHEDULER=0 so that ISL is not invoked per item.")

(define-backend :b200 B200Buffer B200Runtime B200-Renderer B200-Auto-Scheduler t)

(defun item-modules (si)
  "Set of module names that produced the nodes of a Schedule-Item: each JITAble node carries
:_lowering_history = ((GRAPH/<MODULE> . module-node-id) ...) pushed when its module was lowered
(source/api/iseq.lisp:359-361), innermost module first."
  (let ((seen nil))
    (dolist (node (getattr si :items) (nreverse seen))
      (dolist (entry (getattr node :_lowering_history :allow-undefined t))
        (pushnew (car entry) seen)))))

(defun item-has (si &rest module-names)
  (let ((mods (item-modules si)))
    (every #'(lambda (m) (member m mods :test #'string-equal :key #'princ-to-string)) module-names)))

(defun item-op-types (si) (map 'list #'node-type (getattr si :items)))

(defun classify-item (si)
  "-> one of :embedding :layernorm :rmsnorm :linear :relu-matmul :argmax :expr.
The four Linear-shaped kernels of a GPT-2 block, with what the scheduler fuses into them
(source/test-suite/test-schedule.lisp:72-74,128-130):
  c_attn          MATMUL + LINEAR(bias)
  attn.c_proj     MATMUL + LINEAR(bias) + TRANSFORMERBLOCK(residual add)
  mlp.c_fc        MATMUL + LINEAR(bias) + GELU (SIGMOID inside)
  mlp.c_proj      MATMUL + LINEAR(bias) + TRANSFORMERBLOCK(residual add)
  lm_head         MATMUL + LINEAR (no bias)"
  (cond
    ((item-has si "GRAPH/EMBEDDING") :embedding)
    ((item-has si "GRAPH/LAYERNORM") :layernorm)
    ((item-has si "GRAPH/RMSNORM") :rmsnorm)   ; one kernel in the reference too (test-schedule.lisp:164-166)
    ((item-has si "GRAPH/ARGMAXNODE") :argmax)
    ((and (item-has si "GRAPH/MATMUL" "GRAPH/LINEAR")
          (find :WMMA (item-op-types si)))
     :linear)
    ((and (item-has si "GRAPH/MATMUL" "GRAPH/RELU") (find :WMMA (item-op-types si))) :relu-matmul)
    (t :expr)))

(defun linear-epilogue (si)
  "(values activation residual-p bias-p) of a :linear item."
  (values (cond ((item-has si "GRAPH/GELU") +act-gelu+) ((item-has si "GRAPH/RELU") +act-relu+) (t +act-none+))
          (item-has si "GRAPH/TRANSFORMERBLOCK")
          ;; Linear lowers its bias as a separate ADD carrying GRAPH/LINEAR (source/nn/linear.lisp:12-17);
          ;; without a bias the item holds the WMMA alone
          (> (count :ADD (item-op-types si)) (if (item-has si "GRAPH/TRANSFORMERBLOCK") 1 0))))

(defstruct (Plan (:constructor make-plan (kind name args form)))
  kind name args form)

(defmethod print-object ((p Plan) stream)
  (format stream "/* B200 ~(~a~) ~a */" (plan-kind p) (plan-name p)))

(defun item-arg-symbols (si)
  "Argument names of the compiled lambda in call order: storage-id-dst ++ dynamic-shapes ++ storage-id-src
(source/codegen/jit.lisp:131-143)."
  (append (getattr si :storage-id-dst)
          (map 'list #'car (getattr si :dynamic-shapes))
          (getattr si :storage-id-src)))

(defun rows-of (buffer)
  "Product of all but the last dimension of a realised buffer (the M of a Linear / the rows of a LayerNorm)."
  (reduce #'* (butlast (buffer-shape buffer))))

;; ---- callers (run time): take realised buffers, call the C entry point -----------------------------

(defun call-embedding (out ids wte wpe n)
  "[Embedding_Embedding_ADD]: h = wte(tok) + wpe(n + arange(s)) (external/llm/layers.lisp:83-85)."
  (destructuring-bind (b s d) (buffer-shape out)
    (check (foreign-funcall "caten_b200_embed" :pointer *ctx* :pointer (buffer-value ids) :pointer (null-pointer)
                            :pointer (buffer-value wte) :pointer (buffer-value wpe) :pointer (buffer-value out)
                            :int64 b :int64 s :int64 n :int64 d
                            :int64 (first (buffer-shape wte)) :int64 (first (buffer-shape wpe)) :int))))

(defun call-layernorm (out x gamma beta eps)
  (check (foreign-funcall "caten_b200_layernorm" :pointer *ctx* :pointer (buffer-value x) :pointer (buffer-value gamma)
                          :pointer (buffer-value beta) :pointer (buffer-value out)
                          :int64 (rows-of x) :int64 (car (last (buffer-shape x))) :float eps :int)))

(defun call-rmsnorm (out x weight eps)
  "`!rms-norm` (source/nn/normalization.lisp:70-85); weight may be nil."
  (check (foreign-funcall "caten_b200_rmsnorm" :pointer *ctx* :pointer (buffer-value x)
                          :pointer (if weight (buffer-value weight) (null-pointer)) :pointer (buffer-value out)
                          :int64 (rows-of x) :int64 (car (last (buffer-shape x))) :float eps :int)))

(defun call-rope (out x base pos0)
  "`!rope` (source/nn/positional-encoding.lisp:3-56) on x [B S H head-dim]; for hosts that call it as one module-level
operation (the scheduler splits the reference's own lowering into several element-wise items, which run through call-expr)."
  (destructuring-bind (b s h hd) (buffer-shape x)
    (check (foreign-funcall "caten_b200_rope" :pointer *ctx* :pointer (buffer-value x) :pointer (buffer-value out)
                            :int64 b :int64 s :int64 h :int64 hd :float (coerce base 'single-float) :int64 pos0 :int))))

(defun call-linear (out x w bias residual act)
  "y = act(x.W^T + bias) + residual (source/nn/linear.lisp:12-17); the memory planner may have made `out` the
residual's storage, which the kernel allows."
  (check (foreign-funcall "caten_b200_linear" :pointer *ctx* :pointer (weight-handle w) :pointer (buffer-value x)
                          :pointer (if bias (buffer-value bias) (null-pointer))
                          :pointer (if residual (buffer-value residual) (null-pointer))
                          :int act :pointer (buffer-value out) :int64 (rows-of x) :int *precision* :int)))

(defun call-relu-matmul (out a b)
  (destructuring-bind (m k) (last (buffer-shape a) 2)
    (check (foreign-funcall "caten_b200_relu_matmul" :pointer *ctx* :pointer (buffer-value a) :pointer (buffer-value b)
                            :pointer (buffer-value out) :int64 m :int64 k :int64 (car (last (buffer-shape b)))
                            :int *precision* :int))))

(defun call-attention (out qkv k-cache v-cache b s n heads max-seq-len)
  "!assign into the caches + softmax(q.K^T * 0.125 + mask).V of external/llm/layers.lisp:19-51 in one call.
Used by the whole-step path; the per-item path runs the reference's six attention kernels through call-expr."
  (check (foreign-funcall "caten_b200_attention_ex" :pointer *ctx* :pointer (buffer-value qkv)
                          :pointer (buffer-value k-cache) :pointer (buffer-value v-cache) :pointer (buffer-value out)
                          :int64 b :int64 s :int64 n :int64 heads :int64 max-seq-len :int *precision* :int)))

(defun call-argmax (out x)
  (check (foreign-funcall "caten_b200_argmax" :pointer *ctx* :pointer (buffer-value x)
                          :int64 (rows-of x) :int64 (car (last (buffer-shape x))) :pointer (buffer-value out) :int)))

;; ---- generic items: the :EXPR tree as a postfix program for caten_b200_eval_expr ----------------------

(defparameter *opcode*
  '((:LOAD . 1) (:CONST . 2) (:INDEX . 3)
    (:NEG . 10) (:RECIP . 11) (:SIN . 12) (:EXP2 . 13) (:LOG2 . 14) (:SQRT . 15) (:NOT . 16) (:CAST . 17)
    (:ADD . 30) (:MUL . 31) (:MOD . 32) (:IDIV . 33) (:AND . 34) (:OR . 35) (:XOR . 36) (:MAX . 37)
    (:!= . 38) (:< . 39) (:WHERE . 50))
  "CATEN_B200_OP_* of include/caten_b200.h, keyed by the aIR node type (source/aasm/attrs.lisp:42-216).")

(defun value-class (dtype)
  "CATEN_B200_CLS_*: 0 fp32, 1 int32 (int64 buffers are read through int32), 2 bool."
  (cond ((eql dtype :bool) 2) ((dtype/floatp dtype) 0) (t 1)))

(defun buffer-dt (dtype)
  "CATEN_B200_DT_*."
  (ecase dtype (:float32 0) (:int32 1) (:uint32 1) (:int64 2) (:uint64 2) (:uint8 3) (:bool 3)))

(defun word (op arg class) (logior (cdr (assoc op *opcode*)) (ash arg 8) (ash class 16)))

(defun float-bits (x) (float-features:single-float-bits (coerce x 'single-float)))

(defstruct (Program (:constructor %make-program ()))
  (code nil) (consts nil) (operands nil))  ; operands: list of (name . type-relay buffer)

(defun program-const (prg value class)
  (let* ((bits (if (= class 0) (float-bits value) (ldb (byte 32 0) (if (eql value t) 1 (if (null value) 0 (round value))))))
         (pos (or (position bits (program-consts prg))
                  (progn (setf (program-consts prg) (append (program-consts prg) (list bits)))
                         (1- (length (program-consts prg)))))))
    (push (word :CONST pos class) (program-code prg))))

(defun program-load (prg name buffer)
  (let ((pos (or (position name (program-operands prg) :key #'car)
                 (progn (setf (program-operands prg) (append (program-operands prg) (list (cons name buffer))))
                        (1- (length (program-operands prg)))))))
    (push (word :LOAD pos (value-class (buffer-dtype buffer))) (program-code prg))))

(defun compile-expr (prg graph id)
  "Post-order walk of an :EXPR graph (the walk source/codegen/renderer.lisp:331-410 does to print C)."
  (let ((node (id->value graph id)))
    (when (null node) (error "B200: dangling id ~a in an :EXPR" id))
    (let* ((out-type (car (relay-writes (read-type-relay node))))
           (cls (value-class (buffer-dtype out-type))))
      (flet ((kid (i) (compile-expr prg graph (nth i (node-reads node)))))
        (ecase (node-type node)
          (:LOAD (program-const prg (getattr node :value) cls))
          (:AREF (program-load prg (getattr node :storage-id) (getattr node :buffer)))
          ((:MOVE :STORE) (kid 1))
          ((:NEG :RECIP :SIN :EXP2 :LOG2 :SQRT :NOT)
           (kid 0) (push (word (node-type node) 0 cls) (program-code prg)))
          (:CAST
           (kid 1)
           (let ((from (value-class (buffer-dtype (second (relay-reads (read-type-relay node)))))))
             (push (word :CAST from cls) (program-code prg))))
          ((:ADD :MUL :MOD :IDIV :AND :OR :XOR :MAX)
           (kid 0) (kid 1) (push (word (node-type node) 0 cls) (program-code prg)))
          (:WMMA  ; c + a * b
           (kid 0) (kid 1) (kid 2)
           (push (word :MUL 0 cls) (program-code prg)) (push (word :ADD 0 cls) (program-code prg)))
          ((:!= :<)
           (kid 1) (kid 2)
           (push (word (node-type node) 0 (value-class (buffer-dtype (second (relay-reads (read-type-relay node))))))
                 (program-code prg)))
          (:WHERE (kid 0) (kid 1) (kid 2) (push (word :WHERE 0 cls) (program-code prg)))
          (:INDEX-COMPONENTS
           ;; flat index = sum_i stride_i * idx_i over the item's loops
           (let ((strides (cdr (node-reads node))) (first-p t))
             (loop for axis upfrom 0 for stride in strides do
               (push (word :INDEX axis 1) (program-code prg))
               (program-const prg (if (numberp stride) stride (error "B200: symbolic stride in INDEX-COMPONENTS")) 1)
               (push (word :MUL 0 1) (program-code prg))
               (unless first-p (push (word :ADD 0 1) (program-code prg)))
               (setf first-p nil)))))))))

(defcstruct caten-b200-expr
  ;; mirror of `caten_b200_expr` (include/caten_b200.h): 6 loops, 8 operands, 96 code words, 16 constants
  (ndim :int32) (shape :int64 :count 6) (n-reduce :int32) (reduce-op :int32) (accumulate :int32) (n-operands :int32)
  (operand :pointer :count 8) (operand-dtype :int32 :count 8) (operand-offset :int64 :count 8)
  (operand-stride :int64 :count 48)
  (out :pointer) (out-dtype :int32) (out-offset :int64) (out-stride :int64 :count 6)
  (n-code :int32) (code :uint32 :count 96) (consts :uint32 :count 16))

(defun view-offset-and-strides (buffer iteration-space)
  "Element offset and per-loop strides of one operand: index = sum_i stride_i * (from_i + by_i * gid_i)
(source/byoc/clang.lisp:82-99); a broadcast axis has stride 0."
  (let ((offset 0) (strides nil))
    (loop for stride in (iteration-space-strides iteration-space)
          for view in (iteration-space-views iteration-space)
          do (let ((s (if (numberp stride) stride (error "B200: symbolic stride ~a (bind it through :dynamic-shapes first)" stride))))
               (if view
                   (destructuring-bind (from to by broadcast) view
                     (declare (ignore to))
                     (incf offset (* s from))
                     (push (if broadcast 0 (* s by)) strides))
                   (push s strides))))
    (declare (ignorable buffer))
    (values offset (nreverse strides))))

(defun call-expr (prg loop-sizes n-reduce reduce-op accumulate out out-relay out-space operand-buffers operand-spaces)
  "Runs one fused element-wise / reducing item through caten_b200_eval_expr."
  (with-foreign-object (e '(:struct caten-b200-expr))
    (macrolet ((slot (name) `(foreign-slot-value e '(:struct caten-b200-expr) ',name))
               (slot-ptr (name) `(foreign-slot-pointer e '(:struct caten-b200-expr) ',name)))
      (setf (slot ndim) (length loop-sizes) (slot n-reduce) n-reduce (slot reduce-op) reduce-op
            (slot accumulate) (if accumulate 1 0) (slot n-operands) (length operand-buffers))
      (loop for i upfrom 0 for s in loop-sizes do (setf (mem-aref (slot-ptr shape) :int64 i) s))
      (loop for i upfrom 0 for b in operand-buffers for sp in operand-spaces do
        (multiple-value-bind (offset strides) (view-offset-and-strides b sp)
          (setf (mem-aref (slot-ptr operand) :pointer i) (buffer-value b)
                (mem-aref (slot-ptr operand-dtype) :int32 i) (buffer-dt (buffer-dtype b))
                (mem-aref (slot-ptr operand-offset) :int64 i) offset)
          (loop for d upfrom 0 for st in strides do
            (setf (mem-aref (slot-ptr operand-stride) :int64 (+ (* i 6) d)) st))))
      (multiple-value-bind (offset strides) (view-offset-and-strides out out-space)
        (setf (slot out) (buffer-value out) (slot out-dtype) (buffer-dt (buffer-dtype out-relay)) (slot out-offset) offset)
        (loop for d upfrom 0 for st in strides do (setf (mem-aref (slot-ptr out-stride) :int64 d) st)))
      (let ((code (reverse (program-code prg))))
        (assert (<= (length code) 96) () "B200: the item's expression needs ~a words (at most 96)" (length code))
        (assert (<= (length (program-consts prg)) 16) () "B200: more than 16 constants in one item")
        (setf (slot n-code) (length code))
        (loop for i upfrom 0 for w in code do (setf (mem-aref (slot-ptr code) :uint32 i) w))
        (loop for i upfrom 0 for c in (program-consts prg) do (setf (mem-aref (slot-ptr consts) :uint32 i) c))))
    (check (foreign-funcall "caten_b200_eval_expr" :pointer *ctx* :pointer e :int))))

;; ---- %render-kernel / %compile-kernel ------------------------------------------------------------------

(defun find-arg (si predicate)
  "Name of the first source argument whose read-type satisfies predicate."
  (loop for name in (getattr si :storage-id-src)
        for type in (getattr si :read-types)
        if (funcall predicate name type) return name))

(defun plan-linear (si)
  "Roles of a :linear item's sources: W is the rank-2 buffer whose last dimension is the reduced one; x is the
other WMMA operand; bias is rank-1 (broadcast along rows); the residual has the output's shape."
  (let* ((dst (car (getattr si :storage-id-dst)))
         (out-type (car (getattr si :write-types)))
         (out-shape (buffer-shape out-type))
         (srcs (map 'list #'cons (getattr si :storage-id-src) (getattr si :read-types)))
         (w (find-if #'(lambda (p) (and (= 2 (count-if-not #'(lambda (v) (and (listp v) (fourth v))) (buffer-views (cdr p))))
                                        (eql (car (buffer-shape (cdr p))) (car (last out-shape)))))
                     srcs))
         (bias (find-if #'(lambda (p) (and (not (eq p w))
                                           (= 1 (count-if-not #'(lambda (v) (and (listp v) (fourth v))) (buffer-views (cdr p))))))
                        srcs))
         (res (find-if #'(lambda (p) (and (not (eq p w)) (not (eq p bias)) (equal (buffer-shape (cdr p)) out-shape)
                                          (notany #'(lambda (v) (and (listp v) (fourth v))) (buffer-views (cdr p)))))
                       srcs))
         (x (find-if #'(lambda (p) (and (not (eq p w)) (not (eq p bias)) (not (eq p res)))) srcs)))
    (unless (and w x) (error "B200: could not identify the weight and the activation of the Linear item ~a" (getattr si :name)))
    (multiple-value-bind (act residual-p bias-p) (linear-epilogue si)
      (list :out dst :x (car x) :w (car w) :bias (and bias-p bias (car bias)) :res (and residual-p res (car res)) :act act))))

(defmethod %render-kernel ((renderer B200-Renderer) si)
  "Called once per jitable item, possibly from lparallel workers (source/codegen/jit.lisp:387-395): pure, builds a Plan."
  (let* ((kind (classify-item si))
         (args (item-arg-symbols si))
         (dst (car (getattr si :storage-id-dst)))
         (srcs (getattr si :storage-id-src)))
    (make-plan
     kind (getattr si :name) args
     (ecase kind
       (:linear
        (destructuring-bind (&key out x w bias res act) (plan-linear si)
          `(call-linear ,out ,x ,w ,bias ,res ,act)))
       (:relu-matmul `(call-relu-matmul ,dst ,(first srcs) ,(second srcs)))
       (:layernorm
        ;; sources: x, gamma (affine), beta (bias), in graph order (source/nn/normalization.lisp:48-58)
        `(call-layernorm ,dst ,(first srcs) ,(second srcs) ,(third srcs) 1e-5))
       (:embedding
        ;; sources: token ids (float32, apps/gpt2/gpt2.lisp:95), wte, wpe; the start position is the dynamic shape n
        `(call-embedding ,dst ,(first srcs) ,(second srcs) ,(third srcs)
                         ,(or (find 'n (map 'list #'car (getattr si :dynamic-shapes)) :test #'string-equal :key #'symbol-name) 0)))
       (:rmsnorm `(call-rmsnorm ,dst ,(first srcs) ,(second srcs) 1e-5))
       (:argmax `(call-argmax ,dst ,(first srcs)))
       (:expr (plan-expr si))))))

(defun plan-expr (si)
  "Any other item: exactly one loop nest with one :EXPR store (after the optional reduction loops).  Anything else
(several stores, nested control flow) has no kernel here and is refused."
  (let* ((bp (getattr si :blueprint))
         (exprs (remove :EXPR bp :key #'node-type :test-not #'eql))
         (fors (remove :FOR bp :key #'node-type :test-not #'eql)))
    (unless (= 1 (length exprs))
      (error "B200: the item ~a has ~a :EXPR nodes; only single-store items have a kernel (no CPU fallback).~%modules: ~a"
             (getattr si :name) (length exprs) (item-modules si)))
    (let* ((expr-node (car exprs))
           (expr (getattr expr-node :EXPR))
           (prg (%make-program))
           (relay (read-type-relay expr-node)))
      (compile-expr prg (expr-graph expr) (car (node-writes (expr-out expr))))
      `(call-expr
        ',prg
        (list ,@(map 'list #'(lambda (f) (expr->form (getattr f :below))) fors))
        ,(length (getattr si :reduce-dims))
        ,(cond ((null (getattr expr-node :reduction :allow-undefined t)) 0)
               ((find :MAX (map 'list #'node-type (graph-nodes (expr-graph expr)))) 2)
               (t 1))
        ,(and (getattr expr-node :reduction :allow-undefined t) t)
        ,(car (getattr si :storage-id-dst)) ',(car (relay-writes relay)) ',(car (relay-write-iters relay))
        (list ,@(map 'list #'car (program-operands prg)))
        ',(map 'list #'(lambda (p) (find-iteration-space expr-node (car p))) (program-operands prg))))))

(defun expr->form (expr)
  "A loop bound as a Lisp form inside the compiled lambda: a number, or the symbol of a dynamic shape (which is one
of the lambda's arguments).  Bounds that are arithmetic over several symbols are not produced for this path's items."
  (let ((out (expr-out expr)))
    (if (eql (node-type out) :LOAD)
        (getattr out :value)
        (error "B200: loop bound ~a is neither a constant nor a single dynamic shape" expr))))

(defun find-iteration-space (expr-node name)
  "Iteration space (views + strides per loop) of the operand called `name`: the reads of an :EXPR node and the
read iteration spaces of its type relay are parallel lists (source/codegen/shape-inference.lisp:273-304)."
  (loop for read in (node-reads expr-node)
        for space in (relay-read-iters (read-type-relay expr-node))
        if (eql read name) return space))

(defmethod %compile-kernel ((renderer B200-Renderer) items dir)
  "Called once, serially (source/codegen/jit.lisp:520).  No compiler runs: the Plan of every rendered item becomes
(lambda (dst... dynamic-shapes... src...) <call>)."
  (declare (ignore dir))
  (ensure-ctx)
  (dolist (item items)
    (let ((plan (getattr item :rendered-object)))
      (when (typep plan 'Plan)
        (setf (getattr item :compiled-object)
              `(lambda (,@(plan-args plan))
                 (declare (ignorable ,@(plan-args plan)))
                 ,(plan-form plan))))))
  nil)

;;; ~~ whole step: one C call per token ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(defcstruct caten-b200-gpt2-desc
  ;; mirror of `caten_b200_gpt2_desc`
  (n-layers :int32) (d-model :int32) (n-heads :int32) (vocab :int32) (max-seq-len :int32) (batch :int32)
  (eps :float) (precision :int32) (max-rows :int32)
  (wte :pointer) (wpe :pointer) (lnf-g :pointer) (lnf-b :pointer) (lm-head :pointer)
  (ln1-g :pointer) (ln1-b :pointer) (attn-b :pointer) (proj-b :pointer)
  (ln2-g :pointer) (ln2-b :pointer) (fc-b :pointer) (mproj-b :pointer)
  (attn-w :pointer) (proj-w :pointer) (fc-w :pointer) (mproj-w :pointer))

(defun state-dict-buffer (runtime state-dict key)
  "Device buffer of one state-dict entry (keys after remap-state-dict-keys, apps/gpt2/gpt2.lisp:52-80)."
  (let ((tensor (or (gethash key (caten/api:state-dict-entry state-dict)) (error "B200: the state dict has no ~a" key))))
    (->b200-buffer runtime (caten/api:tensor-buffer tensor))))

(defun create-gpt2 (runtime state-dict &key n-layers dim n-heads vocab-size max-seq-len (batch 1) (eps 1e-5))
  "caten_b200_gpt2_create from the uploaded weights.  Replaces, for the GPT-2 Transformer, the :JIT_KERNEL
sequence the VM would walk per token (source/runtime/runtime.lisp:106-145) by one node."
  (flet ((dev (key) (buffer-value (state-dict-buffer runtime state-dict key)))
         (wgt (key) (weight-handle (state-dict-buffer runtime state-dict key))))
    (with-foreign-objects ((d '(:struct caten-b200-gpt2-desc)) (model :pointer))
      (macrolet ((slot (name) `(foreign-slot-value d '(:struct caten-b200-gpt2-desc) ',name)))
        (setf (slot n-layers) n-layers (slot d-model) dim (slot n-heads) n-heads (slot vocab) vocab-size
              (slot max-seq-len) max-seq-len (slot batch) batch (slot eps) eps (slot precision) *precision* (slot max-rows) 0
              (slot wte) (dev "wte.weight") (slot wpe) (dev "wpe.weight")
              (slot lnf-g) (dev "ln_f.affine") (slot lnf-b) (dev "ln_f.bias") (slot lm-head) (wgt "lm_head.weight"))
        (flet ((per-layer (fmt getter)
                 (let ((arr (foreign-alloc :pointer :count n-layers)))
                   (dotimes (l n-layers arr)
                     (setf (mem-aref arr :pointer l) (funcall getter (format nil fmt l)))))))
          (let ((arrays
                  (list
                   (setf (slot ln1-g) (per-layer "h.~a.ln_1.affine" #'dev)) (setf (slot ln1-b) (per-layer "h.~a.ln_1.bias" #'dev))
                   (setf (slot attn-b) (per-layer "h.~a.attn.c_attn.bias" #'dev)) (setf (slot proj-b) (per-layer "h.~a.attn.c_proj.bias" #'dev))
                   (setf (slot ln2-g) (per-layer "h.~a.ln_2.affine" #'dev)) (setf (slot ln2-b) (per-layer "h.~a.ln_2.bias" #'dev))
                   (setf (slot fc-b) (per-layer "h.~a.mlp.c_fc.bias" #'dev)) (setf (slot mproj-b) (per-layer "h.~a.mlp.c_proj.bias" #'dev))
                   (setf (slot attn-w) (per-layer "h.~a.attn.c_attn.weight" #'wgt)) (setf (slot proj-w) (per-layer "h.~a.attn.c_proj.weight" #'wgt))
                   (setf (slot fc-w) (per-layer "h.~a.mlp.c_fc.weight" #'wgt)) (setf (slot mproj-w) (per-layer "h.~a.mlp.c_proj.weight" #'wgt)))))
            (unwind-protect
                 (check (foreign-funcall "caten_b200_gpt2_create" :pointer *ctx* :pointer d :pointer model :int))
              (mapc #'foreign-free arrays)))))   ; the library copies the per-layer tables
      (setf (b200-runtime-gpt2 runtime) (mem-ref model :pointer)
            (b200-runtime-gpt2-batch runtime) batch)
      runtime)))

(defun b200-gpt2-forward (runtime ids-f32 s n)
  "One `(forward model (x . tokens) (s . len) (n . start-pos))` (apps/gpt2/gpt2.lisp:104): ids-f32 is the
single-float vector of batch x s token ids; returns the (signed-byte 64) vector of batch next ids."
  (declare (type (simple-array single-float (*)) ids-f32))
  (let ((out (make-array (b200-runtime-gpt2-batch runtime) :element-type '(signed-byte 64))))
    (with-pointer-to-vector-data (src ids-f32)
      (with-pointer-to-vector-data (dst out)
        (check (foreign-funcall "caten_b200_gpt2_step" :pointer (b200-runtime-gpt2 runtime) :pointer src
                                :int64 s :int64 n :pointer dst :int))))
    out))

;; The peephole: a B200Runtime whose graph is the jitted GPT-2 Transformer answers `forward` with the one call
;; above instead of walking its node list.  make-gpt2-b200 arms it; `gpt2-generate` then runs unchanged, because
;; it only calls (forward model `(x . ,tensor) `(s . ,len) `(n . ,start-pos)) and reads element 0 of the result.
(defmethod caten/api:forward :around ((runtime B200Runtime) &rest params)
  (if (null (b200-runtime-gpt2 runtime))
      (call-next-method)
      (flet ((param (name)
               (let ((hit (find name params :test #'string-equal :key #'(lambda (p) (symbol-name (car p))))))
                 (or (cdr hit) (error "B200: forward needs the parameter ~a" name)))))
        (let* ((x (param "X")) (s (param "S")) (n (param "N"))
               (ids (caten/api:change-facet x :simple-array))
               (out (b200-gpt2-forward runtime (coerce ids '(simple-array single-float (*))) s n)))
          (caten/api:change-facet (list (coerce out 'list)) :tensor)))))

(defun make-gpt2-b200 (model-type gguf-path &key (max-seq-len 1024) (batch 1))
  "The batched variant of `make-gpt2` (apps/gpt2/gpt2.lisp:82-93, which hard-wires batch 1 at :93): loads the file
with the packed-weight loader, remaps the keys and builds the device model.  Returns the runtime; wrap it with
caten/apps.gpt2::%make-gpt2 and a tokenizer to drive `gpt2-generate`."
  (ctx:with-contextvar (:BACKEND "B200")
    (let* ((param (caten/apps.gpt2::get-param model-type))
           (gguf (caten/gguf:load-gguf gguf-path))
           (state-dict (caten/gguf:gguf->state-dict gguf))
           (runtime (caten/api:get-global-runtime)))
      (caten/apps.gpt2::remap-state-dict-keys state-dict)
      (create-gpt2 (make-runtime (make-graph) :runtime 'B200Runtime :buffer-type 'B200Buffer)
                   state-dict
                   :n-layers (caten/apps.gpt2::params-n-layers param) :dim (caten/apps.gpt2::params-dim param)
                   :n-heads (caten/apps.gpt2::params-n-heads param) :vocab-size (caten/apps.gpt2::params-vocab-size param)
                   :eps (caten/apps.gpt2::params-norm-eps param) :max-seq-len max-seq-len :batch batch)
      runtime)))

;;; ~~ multi-GPU: one Lisp image per GPU ~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~~

(defun dist-unique-id ()
  "Rank 0: a fresh 128-byte group id to hand to the other ranks (a file, the environment, a socket)."
  (ensure-ctx)
  (let ((id (make-array +dist-id-bytes+ :element-type '(unsigned-byte 8))))
    (with-pointer-to-vector-data (p id)
      (check (foreign-funcall "caten_b200_dist_unique_id" :pointer p :int)))
    id))

(defun dist-init (rank world id)
  (with-pointer-to-vector-data (p id)
    (check (foreign-funcall "caten_b200_dist_init" :pointer (ensure-ctx) :int rank :int world :pointer p :int))))

(defun dist-shard (batch world rank)
  "(values first count): the contiguous slice of the batch this rank owns."
  (with-foreign-objects ((first :int64) (count :int64))
    (check (foreign-funcall "caten_b200_dist_shard" :int64 batch :int world :int rank :pointer first :pointer count :int))
    (values (mem-ref first :int64) (mem-ref count :int64))))

(defun dist-bcast-weights (device-arena nbytes &optional (root 0))
  "Rank `root` holds the file's tensor data at device-arena; afterwards every rank does, and uploads its weights from it
with caten_b200_weight_upload_device."
  (check (foreign-funcall "caten_b200_dist_bcast_weights" :pointer *ctx* :pointer device-arena :size nbytes :int root :int)))

(defun dist-gather-ids (device-local n-per-rank device-all)
  (check (foreign-funcall "caten_b200_dist_gather_ids" :pointer *ctx* :pointer device-local :int64 n-per-rank
                          :pointer device-all :int)))

(defun dist-finalize ()
  (check (foreign-funcall "caten_b200_dist_finalize" :pointer *ctx* :int)))
