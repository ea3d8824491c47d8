;; The keyword-level API over the raw calls of impl.clj: descriptors from shapes and layout
;; keywords, scalars cast to the tensor's compute type, handles and buffers unwrapped.  The
;; counterpart of uncomplicate.diamond.internal.cudnn.core (deep-diamond-cuda,
;; src/clojure/uncomplicate/diamond/internal/cudnn/core.clj:48-231 and :344-350), with the same
;; function names and argument orders, so that tensor.clj / factory.clj / directed.clj of a B200
;; backend are the cuDNN ones with the namespace swapped.
;; NOT EXECUTED where it was written (no JVM there).

(ns uncomplicate.diamond.internal.b200.core
  (:require [uncomplicate.commons
             [core :refer [let-release with-release release]]
             [utils :refer [dragan-says-ex enc-keyword]]]
            [uncomplicate.fluokitten.protocols :refer [extract]]
            [uncomplicate.diamond.internal.b200
             [protocols :refer :all]
             [constants :refer :all]
             [impl :refer :all]])
  (:import java.lang.foreign.Arena
           [uncomplicate.diamond.internal.b200.impl B200TensorDescriptor]))

;; =========================== Handle ====================================================

(defn b200-context
  "A library handle on `stream` (a ClojureCUDA stream); the current CUDA context's device must be a
  B200 (cudnn-context, cudnn/core.clj:41-47)."
  [stream]
  (b200-context* (extract stream)))

(defn get-b200-stream [handle]
  (get-b200-stream* handle))

;; =========================== Tensor descriptor =========================================

(defn- default-strides [shape]
  (vec (rest (reductions (fn [^long acc ^long d] (quot acc (max 1 d)))
                         (reduce * 1 (map #(max 1 (long %)) shape))
                         shape))))

(defn tensor-descriptor
  "`layout` is :nchw / :nhwc (ranks up to 8: the named layout of the trailing dims) or a stride
  vector.  Ranks 1-8 are native: no padding of short shapes to rank 4 (cudnn-tensor-desc,
  cudnn/tensor.clj:119-131, is not needed).  After tensor-descriptor, cudnn/core.clj:48-70."
  [shape data-type layout]
  (let [dtype (enc-keyword dd-data-type data-type)
        td (tensor-descriptor*)]
    (try
      (wrap-tensor-struct
       (cond
         (keyword? layout)
         (tensor-nd-descriptor-ex* td (enc-keyword dd-format layout) dtype (vec shape))
         (nil? layout)
         (tensor-nd-descriptor* td dtype (vec shape) (default-strides shape))
         (= (count shape) (count layout))
         (tensor-nd-descriptor* td dtype (vec shape) (vec layout))
         :default
         (dragan-says-ex "Shape and strides must have the same length."
                         {:shape shape :strides layout})))
      (catch Exception e
        (destroy-tensor-descriptor* td)
        (throw e)))))

(defn equal-desc?
  "Structural equality of two descriptor providers (cudnn/core.clj:72-78)."
  [td1 td2]
  (= (desc td1) (desc td2)))

(defn data-type [td]
  (.data-type ^B200TensorDescriptor (desc td)))

(defn dims [td]
  (.dims ^B200TensorDescriptor (desc td)))

(defn ndims ^long [td]
  (count (dims td)))

(defn strides [td]
  (.layout ^B200TensorDescriptor (desc td)))

(defn size-in-bytes ^long [td]
  (tensor-size-in-bytes* (extract (desc td))))

;; =========================== Set, scale, add, reorder ==================================

(defmacro ^:private with-scalars
  "Binds each symbol to a host cell holding its value in the compute type of `dtype`."
  [dtype syms & body]
  `(with-open [arena# (Arena/ofConfined)]
     (let [~@(mapcat (fn [s] [s `(scalar-seg arena# ~dtype ~s)]) syms)]
       ~@body)))

(defn set-tensor
  "x[:] = value (cudnn/core.clj:100-106)."
  [handle desc-x x value]
  (with-scalars (data-type desc-x) [value]
    (set-tensor* handle (extract (desc desc-x)) x value))
  handle)

(defn scale-tensor
  "x *= alpha (cudnn/core.clj:108-115)."
  [handle alpha desc-x x]
  (with-scalars (data-type desc-x) [alpha]
    (scale-tensor* handle (extract (desc desc-x)) x alpha))
  handle)

(defn add-tensor
  "y = alpha * broadcast(x) + beta * y; every dim of x is 1 or y's (cudnn/core.clj:117-129)."
  [handle alpha desc-x x beta desc-y y]
  (with-scalars (data-type desc-y) [alpha beta]
    (add-tensor* handle alpha (extract (desc desc-x)) x beta (extract (desc desc-y)) y))
  handle)

(defn op-tensor
  "c = op(alpha1 * a, alpha2 * broadcast(b)) + beta * c, op one of :add :mul :min :max :sub :div
  (the GPU form of the DNNL backend's `binary`, dnnl/core.clj:430-447)."
  [handle op alpha1 desc-a a alpha2 desc-b b beta desc-c c]
  (with-scalars (data-type desc-c) [alpha1 alpha2 beta]
    (op-tensor* handle (enc-keyword dd-op-tensor-op op)
                alpha1 (extract (desc desc-a)) a alpha2 (extract (desc desc-b)) b
                beta (extract (desc desc-c)) c))
  handle)

(defn sum-tensors
  "dst = sum of scales[i] * srcs[i] in one pass (the DNNL backend's `sum!`, dnnl/core.clj:392-426;
  on cuDNN it is a loop of axpy!, cudnn/directed.clj:1762-1766)."
  [handle scales descs srcs desc-dst dst]
  (sum-tensors* handle scales (mapv #(extract (desc %)) descs) srcs (extract (desc desc-dst)) dst)
  handle)

(defn transform-tensor
  "y = alpha * convert(x) + beta * y over equal shapes, any strides, any pair of data types
  (cudnn/core.clj:131-144)."
  [handle alpha desc-x buf-x beta desc-y buf-y]
  (with-scalars (data-type desc-y) [alpha beta]
    (transform-tensor* handle alpha (extract (desc desc-x)) buf-x beta (extract (desc desc-y)) buf-y))
  handle)

(defn gather-transform
  "One launch that copies (and converts) `(count src-offsets)` sub-tensors: what a shuffler does
  with one batcher call per column (cudnn/tensor.clj:306-317)."
  [handle src-offsets dst-offsets sub-desc-x buf-x sub-desc-y buf-y]
  (gather-transform* handle (vec src-offsets) (vec dst-offsets)
                     (extract (desc sub-desc-x)) buf-x (extract (desc sub-desc-y)) buf-y)
  handle)

(defn multi-transform
  "Up to 8 (source, destination) sub-tensor copies in one launch: the transformer loops of the
  branch and concatenate layers (cudnn/directed.clj:1331-1333,1402-1409).  `pairs` is a sequence of
  [desc-x buf-x desc-y buf-y]."
  [handle pairs]
  (multi-transform* handle
                    (mapv #(extract (desc (nth % 0))) pairs) (mapv #(nth % 1) pairs)
                    (mapv #(extract (desc (nth % 2))) pairs) (mapv #(nth % 3) pairs))
  handle)

(defn cost-diff
  "d = a - y and, in the same pass, the cost of `kind` (:quadratic, :mean-absolute, :crossentropy)
  into the device double `cost` (cudnn/directed.clj:367-412 does it with axpy! and nrm2 / asum)."
  [handle kind desc-a a y d cost]
  (cost-diff* handle (enc-keyword dd-cost-kind kind) (extract (desc desc-a)) a y d cost)
  handle)

(defn tensor-equals
  "Sets the device int `flag` to 1 when any element differs (equals-block, cudnn/factory.clj:123-133)."
  [handle desc-x x desc-y y flag]
  (tensor-equals* handle (extract (desc desc-x)) x (extract (desc desc-y)) y flag)
  handle)

;; =========================== Activation ================================================

(defn activation-descriptor
  "After activation-descriptor, cudnn/core.clj:148-164; `shift` is the beta of :linear."
  ([mode relu-nan-opt ^double coef ^double shift]
   (let [ad (activation-descriptor*)]
     (try
       (activation-descriptor* ad (enc-keyword dd-activation-mode mode)
                               (enc-nan-propagation relu-nan-opt) coef shift)
       (catch Exception e
         (destroy-activation-descriptor* ad)
         (throw e)))))
  ([mode relu-nan-opt ^double coef]
   (activation-descriptor mode relu-nan-opt coef 0.0))
  ([mode ^double coef]
   (activation-descriptor mode true coef 0.0))
  ([ad]
   (let [{:keys [mode relu-nan-opt coef]} (get-activation-descriptor* ad)]
     {:mode (dec-activation-mode mode)
      :relu-nan-opt (dec-nan-propagation relu-nan-opt)
      :coef coef})))

(defn activation-forward
  "y = alpha * act(x) + beta * y (cudnn/core.clj:166-172)."
  [handle ad alpha desc-x buf-x beta desc-y buf-y]
  (with-scalars (data-type desc-y) [alpha beta]
    (activation-forward* handle ad alpha (extract (desc desc-x)) buf-x beta (extract (desc desc-y)) buf-y))
  handle)

(defn activation-backward
  "dx = alpha * act'(x) * dy + beta * dx, the derivative taken from x like the DNNL backend
  (dnnl/core.clj:382-388); `buf-y` is accepted and not read (cudnn/core.clj:174-184)."
  [handle ad alpha desc-y buf-y desc-dy buf-dy desc-x buf-x beta desc-dx buf-dx]
  (with-scalars (data-type desc-dx) [alpha beta]
    (activation-backward* handle ad alpha (extract (desc desc-y)) buf-y
                          (extract (desc desc-dy)) buf-dy (extract (desc desc-x)) buf-x
                          beta (extract (desc desc-dx)) buf-dx))
  handle)

;; =========================== Reduce ====================================================

(defn reduce-tensor-descriptor
  "After reduce-tensor-descriptor, cudnn/core.clj:188-205: the 4-argument arity is the reference's
  (op comp-type nan-opt indices), :flattened asking min / max / amax for the positions too.  The
  5-argument arity carries the p and epsilon of the DNNL backend's `reduction`
  (dnnl/core.clj:796-803) for the :norm-lp-* kinds."
  ([op comp-type nan-opt p eps]
   (let [rtd (reduce-tensor-descriptor*)]
     (try
       (reduce-tensor-descriptor* rtd (enc-keyword dd-reduce-tensor-op op)
                                  (enc-keyword dd-data-type comp-type)
                                  (enc-nan-propagation nan-opt)
                                  (double p) (double eps))
       (catch Exception e
         (destroy-reduce-tensor-descriptor* rtd)
         (throw e)))))
  ([op comp-type nan-opt indices]
   (let [rtd (reduce-tensor-descriptor op comp-type nan-opt)]
     (try
       (reduce-tensor-descriptor-indices* rtd (enc-keyword dd-reduce-tensor-indices indices))
       (catch Exception e
         (destroy-reduce-tensor-descriptor* rtd)
         (throw e)))))
  ([op comp-type nan-opt]
   (let [rtd (reduce-tensor-descriptor*)]
     (try
       (reduce-tensor-descriptor* rtd (enc-keyword dd-reduce-tensor-op op)
                                  (enc-keyword dd-data-type comp-type)
                                  (enc-nan-propagation nan-opt))
       (catch Exception e
         (destroy-reduce-tensor-descriptor* rtd)
         (throw e)))))
  ([op comp-type]
   (reduce-tensor-descriptor op comp-type true)))

(defn reduction-indices-size ^long [handle rtd desc-x desc-y]
  (reduction-indices-size* handle rtd (extract (desc desc-x)) (extract (desc desc-y))))

(defn reduction-workspace-size ^long [handle rtd desc-x desc-y]
  (reduction-workspace-size* handle rtd (extract (desc desc-x)) (extract (desc desc-y))))

(defn reduce-tensor
  "y = alpha * reduce(x) + beta * y over the dims where y's extent is 1.  The 8-argument arity uses
  the handle's own scratch: no cuda-malloc / cuda-free! per call (cudnn/core.clj:213-231 does two)."
  ([handle rtd workspace ^long workspace-size alpha desc-x buf-x beta desc-y buf-y]
   (with-scalars (data-type desc-y) [alpha beta]
     (reduce-tensor* handle rtd nil 0 workspace workspace-size
                     alpha (extract (desc desc-x)) buf-x beta (extract (desc desc-y)) buf-y))
   handle)
  ([handle rtd alpha desc-x buf-x beta desc-y buf-y]
   (reduce-tensor handle rtd nil 0 alpha desc-x buf-x beta desc-y buf-y)))

(defn convolution-bwd-bias
  "db = alpha * (sum of dy over the dims where db's extent is 1) + beta * db
  (cudnn/core.clj:344-350)."
  [handle alpha desc-dy buf-dy beta desc-db buf-db]
  (with-scalars (data-type desc-db) [alpha beta]
    (convolution-bwd-bias* handle alpha (extract (desc desc-dy)) buf-dy beta (extract (desc desc-db)) buf-db))
  handle)

;; =========================== More than one GPU =========================================

(defn sharded-reduce-tensor
  "Collective over the ranks of `sh`: `desc-x` is this rank's shard, y is replicated.
  `global-count` is the number of elements folded into one output over all ranks (0: equal shards)."
  [handle sh rtd spans? global-count alpha desc-x buf-x beta desc-y buf-y]
  (with-scalars (data-type desc-y) [alpha beta]
    (sharded-reduce-tensor* handle sh rtd spans? (long global-count)
                            alpha (extract (desc desc-x)) buf-x beta (extract (desc desc-y)) buf-y))
  handle)

(defn sharded-release
  "The collective tear-down: detach, meet the other ranks at `barrier!` (a function of no
  arguments over the host's own transport), then free what this rank exported."
  [sh barrier!]
  (sharded-peer-detach* sh)
  (barrier!)
  (sharded-destroy* sh))
