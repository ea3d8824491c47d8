;; Keyword <-> enum tables of libdd_b200.so (include/dd_b200.h).  The counterpart of
;; uncomplicate.diamond.internal.cudnn.constants (deep-diamond-cuda,
;; src/clojure/uncomplicate/diamond/internal/cudnn/constants.clj): the same keywords, so that
;; core.clj, tensor.clj and factory.clj read alike, with the numbers this library defines.
;; NOT EXECUTED where it was written (no JVM there); tests/test_clojure_binding.py compares every
;; number below with the header's enums.

(ns uncomplicate.diamond.internal.b200.constants
  (:require [uncomplicate.commons.utils :refer [dragan-says-ex]]))

(def ^:const dd-dim-max 8)
(def ^:const dd-unique-id-bytes 128)
(def ^:const dd-peer-handle-bytes 64)
(def ^:const dd-handle-scratch-bytes (* 8 1024 1024))
(def ^:const dd-noalloc-scratch-bytes (* 64 1024))

(def ^{:const true
       :doc "Status codes of the library; 0-9 carry cuDNN's keywords (cudnn/constants.clj:16-33)."}
  dd-status-codes
  {0 :success
   1 :not-initialized
   2 :alloc-failed
   3 :bad-param
   4 :internal-error
   5 :invalid-value
   6 :arch-mismatch
   7 :mapping-error
   8 :execution-failed
   9 :not-supported
   10 :timeout
   11 :comm-failed})

(defn enc-nan-propagation ^long [nan]
  (if nan 1 0))

(defn dec-nan-propagation [^long nan]
  (= 1 nan))

(def ^{:const true
       :doc "Named layouts (cudnn/constants.clj:43-55); every other layout travels as strides."}
  dd-format
  {:nchw 0
   :nhwc 1
   :abcd 0
   :acdb 1
   :oihw 0
   :ohwi 1})

(defn dec-format [^long format]
  (case format
    0 :nchw
    1 :nhwc
    (dragan-says-ex "This format is not supported by libdd_b200." {:format format})))

(def ^{:const true
       :doc "Data types: cuDNN's codes for the types it has (cudnn/constants.clj:64-89), 9 for
  bfloat16 and 15 for int64."}
  dd-data-type
  {:float 0
   :float32 0
   :f32 0
   Float/TYPE 0
   Float 0
   :double 1
   :float64 1
   :f64 1
   Double/TYPE 1
   Double 1
   :half 2
   :float16 2
   :f16 2
   :byte 3
   :int8 3
   :s8 3
   Byte/TYPE 3
   Byte 3
   :int 4
   :int32 4
   :s32 4
   Integer/TYPE 4
   Integer 4
   :uint8 6
   :u8 6
   :bf16 9
   :bfloat16 9
   :long 15
   :int64 15
   :s64 15
   Long/TYPE 15
   Long 15})

(defn dec-data-type [^long data-type]
  (case data-type
    0 :float
    1 :double
    2 :half
    3 :byte
    4 :int
    6 :uint8
    9 :bf16
    15 :long
    (dragan-says-ex "This data type is not supported by libdd_b200."
                    {:data-type data-type :available (keys dd-data-type)})))

(defn data-type-width ^long [data-type]
  (case (dec-data-type (long (get dd-data-type data-type -1)))
    :float 4
    :double 8
    :half 2
    :byte 1
    :int 4
    :uint8 1
    :bf16 2
    :long 8))

(def ^{:const true
       :doc "Activation modes: cuDNN's (cudnn/constants.clj:150-158) plus the kinds of the DNNL
  backend's table (dnnl/constants.clj:277-308; like that table, :square-dst-bwd maps onto oneDNN's
  sqrt_use_dst_for_bwd).  :linear / :identity is a real mode here."}
  dd-activation-mode
  {:logistic 0
   :sigmoid 0
   :relu 1
   :tanh 2
   :clipped-relu 3
   :elu 4
   :linear 5
   :identity 5
   :abs 6
   :square 7
   :sqrt 8
   :exp 9
   :log 10
   :soft-relu 11
   :swish 12
   :gelu 13
   :gelu-tanh 13
   :gelu-erf 14
   :hardswish 15
   :clip 16
   :clip-v2 17
   :pow 18
   :mish 19
   :round 20
   :relu-dst-bwd 21
   :tanh-dst-bwd 22
   :elu-dst-bwd 23
   :square-dst-bwd 24
   :sqrt-dst-bwd 24
   :logistic-dst-bwd 25
   :sigmoid-dst-bwd 25
   :exp-dst-bwd 26
   :clip-v2-dst-bwd 27})

(defn dec-activation-mode [^long mode]
  (case mode
    0 :logistic
    1 :relu
    2 :tanh
    3 :clipped-relu
    4 :elu
    5 :linear
    6 :abs
    7 :square
    8 :sqrt
    9 :exp
    10 :log
    11 :soft-relu
    12 :swish
    13 :gelu-tanh
    14 :gelu-erf
    15 :hardswish
    16 :clip
    17 :clip-v2
    18 :pow
    19 :mish
    20 :round
    21 :relu-dst-bwd
    22 :tanh-dst-bwd
    23 :elu-dst-bwd
    24 :sqrt-dst-bwd
    25 :logistic-dst-bwd
    26 :exp-dst-bwd
    27 :clip-v2-dst-bwd
    (dragan-says-ex "This mode is not supported by libdd_b200."
                    {:mode mode :available (keys dd-activation-mode)})))

(def ^{:const true
       :doc "Binary ops of ddOpTensor: cudnnOpTensor's four and the kinds of oneDNN's binary
  primitive (dnnl/constants.clj:359-371), comparisons included (1 / 0 in the tensors' type)."}
  dd-op-tensor-op
  {:add 0
   :mul 1
   :min 2
   :max 3
   :sub 4
   :div 5
   :ge 6
   :gt 7
   :le 8
   :lt 9
   :eq 10
   :ne 11})

(def ^{:const true
       :doc "Reduce ops (cudnn/constants.clj:171-180) with oneDNN's names accepted too
  (dnnl/constants.clj:393-402)."}
  dd-reduce-tensor-op
  {:add 0
   :sum 0
   :mul 1
   :min 2
   :max 3
   :amax 4
   :avg 5
   :mean 5
   :norm1 6
   :norm2 7
   :mul-no-zeros 8
   :norm-lp-max 9
   :norm-lp-sum 10
   :norm-lp-power-p-max 11
   :norm-lp-power-p-sum 12})

(def ^{:const true
       :doc "cudnn/constants.clj:182-184."}
  dd-reduce-tensor-indices
  {:no-indices 0
   :flattened 1})

(defn dec-reduce-tensor-op [^long op]
  (case op
    0 :add
    1 :mul
    2 :min
    3 :max
    4 :amax
    5 :avg
    6 :norm1
    7 :norm2
    8 :mul-no-zeros
    9 :norm-lp-max
    10 :norm-lp-sum
    11 :norm-lp-power-p-max
    12 :norm-lp-power-p-sum
    (dragan-says-ex "This reduce op is not supported by libdd_b200."
                    {:op op :available (keys dd-reduce-tensor-op)})))

(def ^{:const true
       :doc "Cost kinds of ddCostDiff."}
  dd-cost-kind
  {:quadratic 0
   :mean-absolute 1
   :crossentropy 2})

(def ^{:const true
       :doc "Forms of the cross-GPU combine step (ddShardedPeerConfigure)."}
  dd-peer-mode
  {:keep -1
   :nccl 0
   :peer 1
   :peer-fused 2
   :peer-separate 3})
