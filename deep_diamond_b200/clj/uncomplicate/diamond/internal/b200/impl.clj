;; Raw binding of libdd_b200.so for a Deep Diamond backend: one downcall handle per exported C
;; function (include/dd_b200.h) and one `*`-suffixed function per call that checks the status.
;; The counterpart of uncomplicate.diamond.internal.cudnn.impl (deep-diamond-cuda,
;; src/clojure/uncomplicate/diamond/internal/cudnn/impl.clj), with the JDK's foreign function API
;; (java.lang.foreign, JDK 22+) in the place of the JavaCPP cuDNN preset.
;;
;; NOT EXECUTED where it was written: that machine has no JVM.  tests/test_clojure_binding.py checks
;; every `defdowncall` below (name, argument count, argument kinds, result kind) against the header
;; and against the symbols the built library exports.
;;
;; Conventions: a handle, a descriptor, a device buffer and a host out-parameter all travel as
;; MemorySegment (layout ADDRESS).  `seg` turns what the rest of Deep Diamond holds (a ClojureCUDA /
;; clojure-cpp pointer, a raw address, nil) into one.  alpha / beta / value are host scalars of the
;; tensor's compute type: float, or double for :double tensors (cudnn/core.clj:139-140 passes
;; `(pointer alpha)` the same way).

(ns uncomplicate.diamond.internal.b200.impl
  (:require [uncomplicate.commons.core :refer [Releaseable release Info info]]
            [uncomplicate.commons.utils :refer [dragan-says-ex]]
            [uncomplicate.fluokitten.protocols :refer [Comonad extract]]
            [uncomplicate.clojure-cpp :as cpp]
            [uncomplicate.diamond.internal.b200
             [constants :refer :all]
             [protocols :refer :all]])
  (:import [java.lang.foreign Arena FunctionDescriptor Linker Linker$Option MemoryLayout MemorySegment
            SymbolLookup ValueLayout]
           java.lang.invoke.MethodHandle))

;; =========================== Loading ===================================================

(def ^:private ^Linker linker (Linker/nativeLinker))

(def ^:private library-name
  (or (System/getProperty "uncomplicate.diamond.b200.library")
      (System/getenv "DD_B200_LIBRARY")
      "libdd_b200.so"))

(def ^:private ^SymbolLookup library
  (SymbolLookup/libraryLookup ^String library-name (Arena/global)))

(def ^:private I ValueLayout/JAVA_INT)
(def ^:private L ValueLayout/JAVA_LONG)
(def ^:private D ValueLayout/JAVA_DOUBLE)
(def ^:private P ValueLayout/ADDRESS)

(defn- downcall ^MethodHandle [^String c-name res args]
  (let [sym (.orElseThrow (.find library c-name))
        fd (FunctionDescriptor/of ^MemoryLayout res (into-array MemoryLayout args))]
    (.downcallHandle linker sym fd (make-array Linker$Option 0))))

(defmacro ^:private defdowncall
  "Defines `clj-name` as the downcall handle of the C function `c-name` with result layout `res`
  (I int / enum, L int64_t / size_t / uint64_t, D double, P any pointer) and argument layouts `args`."
  [clj-name c-name res args]
  `(def ~(vary-meta clj-name assoc :private true :tag `MethodHandle) (downcall ~c-name ~res ~args)))

(defdowncall dd-create                            "ddCreate" I [P])
(defdowncall dd-destroy                           "ddDestroy" I [P])
(defdowncall dd-set-stream                        "ddSetStream" I [P P])
(defdowncall dd-get-stream                        "ddGetStream" I [P P])
(defdowncall dd-get-error-string                  "ddGetErrorString" P [I])
(defdowncall dd-get-last-error-message            "ddGetLastErrorMessage" P [P])
(defdowncall dd-get-version                       "ddGetVersion" L [])
(defdowncall dd-get-launch-count                  "ddGetLaunchCount" I [P P])
(defdowncall dd-get-last-kernel-name              "ddGetLastKernelName" P [P])
(defdowncall dd-reset-counters                    "ddResetCounters" I [P])
(defdowncall dd-get-device-fault                  "ddGetDeviceFault" I [P P])
(defdowncall dd-create-tensor-descriptor          "ddCreateTensorDescriptor" I [P])
(defdowncall dd-destroy-tensor-descriptor         "ddDestroyTensorDescriptor" I [P])
(defdowncall dd-set-tensor4d-descriptor           "ddSetTensor4dDescriptor" I [P I I L L L L])
(defdowncall dd-set-tensor4d-descriptor-ex        "ddSetTensor4dDescriptorEx" I [P I L L L L L L L L])
(defdowncall dd-set-tensor-nd-descriptor          "ddSetTensorNdDescriptor" I [P I I P P])
(defdowncall dd-set-tensor-nd-descriptor-ex       "ddSetTensorNdDescriptorEx" I [P I I I P])
(defdowncall dd-get-tensor-nd-descriptor          "ddGetTensorNdDescriptor" I [P I P P P P])
(defdowncall dd-get-tensor-size-in-bytes          "ddGetTensorSizeInBytes" I [P P])
(defdowncall dd-set-tensor                        "ddSetTensor" I [P P P P])
(defdowncall dd-scale-tensor                      "ddScaleTensor" I [P P P P])
(defdowncall dd-add-tensor                        "ddAddTensor" I [P P P P P P P])
(defdowncall dd-op-tensor                         "ddOpTensor" I [P I P P P P P P P P P])
(defdowncall dd-sum-tensors                       "ddSumTensors" I [P I P P P P P])
(defdowncall dd-transform-tensor                  "ddTransformTensor" I [P P P P P P P])
(defdowncall dd-gather-transform                  "ddGatherTransform" I [P I P P P P P P])
(defdowncall dd-tensor-equals                     "ddTensorEquals" I [P P P P P P])
(defdowncall dd-multi-transform                   "ddMultiTransform" I [P I P P P P])
(defdowncall dd-cost-diff                         "ddCostDiff" I [P I P P P P P])
(defdowncall dd-create-activation-descriptor      "ddCreateActivationDescriptor" I [P])
(defdowncall dd-destroy-activation-descriptor     "ddDestroyActivationDescriptor" I [P])
(defdowncall dd-set-activation-descriptor         "ddSetActivationDescriptor" I [P I I D])
(defdowncall dd-set-activation-descriptor-ex      "ddSetActivationDescriptorEx" I [P I I D D])
(defdowncall dd-get-activation-descriptor         "ddGetActivationDescriptor" I [P P P P])
(defdowncall dd-activation-forward                "ddActivationForward" I [P P P P P P P P])
(defdowncall dd-activation-backward               "ddActivationBackward" I [P P P P P P P P P P P P])
(defdowncall dd-create-reduce-tensor-descriptor   "ddCreateReduceTensorDescriptor" I [P])
(defdowncall dd-destroy-reduce-tensor-descriptor  "ddDestroyReduceTensorDescriptor" I [P])
(defdowncall dd-set-reduce-tensor-descriptor      "ddSetReduceTensorDescriptor" I [P I I I])
(defdowncall dd-get-reduce-tensor-descriptor      "ddGetReduceTensorDescriptor" I [P P P P])
(defdowncall dd-set-reduce-tensor-descriptor-lp   "ddSetReduceTensorDescriptorLp" I [P I I I D D])
(defdowncall dd-get-reduce-tensor-descriptor-lp   "ddGetReduceTensorDescriptorLp" I [P P P])
(defdowncall dd-set-reduce-tensor-descriptor-indices "ddSetReduceTensorDescriptorIndices" I [P I])
(defdowncall dd-get-reduction-indices-size        "ddGetReductionIndicesSize" I [P P P P P])
(defdowncall dd-get-reduction-workspace-size      "ddGetReductionWorkspaceSize" I [P P P P P])
(defdowncall dd-reduce-tensor                     "ddReduceTensor" I [P P P L P L P P P P P P])
(defdowncall dd-convolution-backward-bias         "ddConvolutionBackwardBias" I [P P P P P P P])
(defdowncall dd-reduce-tensor-no-alloc            "ddReduceTensorNoAlloc" I [P I I P P P P P P P L])
(defdowncall dd-sharded-get-unique-id             "ddShardedGetUniqueId" I [P])
(defdowncall dd-sharded-set-join-limit            "ddShardedSetJoinLimit" I [D])
(defdowncall dd-sharded-create                    "ddShardedCreate" I [P P I I P])
(defdowncall dd-sharded-peer-detach               "ddShardedPeerDetach" I [P])
(defdowncall dd-sharded-destroy                   "ddShardedDestroy" I [P])
(defdowncall dd-sharded-reduce-tensor             "ddShardedReduceTensor" I [P P I L P P P P P P])
(defdowncall dd-sharded-peer-export               "ddShardedPeerExport" I [P P])
(defdowncall dd-sharded-peer-attach               "ddShardedPeerAttach" I [P P])
(defdowncall dd-sharded-peer-configure            "ddShardedPeerConfigure" I [P I D])
(defdowncall dd-sharded-peer-status               "ddShardedPeerStatus" I [P P])
(defdowncall dd-sharded-check                     "ddShardedCheck" I [P])

;; =========================== Calling ===================================================

(defn seg
  "The MemorySegment a C pointer argument needs: nil -> NULL, a MemorySegment as is, a long as a raw
  address, anything else (ClojureCUDA device pointers, clojure-cpp host pointers) by its address."
  ^MemorySegment [x]
  (cond
    (nil? x) MemorySegment/NULL
    (instance? MemorySegment x) x
    (integer? x) (MemorySegment/ofAddress (long x))
    :else (MemorySegment/ofAddress (long (cpp/address (cpp/ptr x))))))

(defn- invoke [^MethodHandle mh & args]
  (.invokeWithArguments mh ^java.util.List (vec args)))

(defn- c-string [^MemorySegment s]
  (if (= 0 (.address s)) "" (.getString (.reinterpret s 512) 0)))

(defn b200-error
  "The ex-info of a non-zero status: {:name :code :type :details}, after cudnn-error
  (cudnn/impl.clj:30-33)."
  [^long err-code hdl details]
  (let [err (get dd-status-codes err-code err-code)]
    (ex-info (format "libdd_b200 error: %s." (name err))
             {:name err :code err-code :type :b200-error
              :message (if hdl (c-string (invoke dd-get-last-error-message (seg hdl))) "")
              :details details})))

(defmacro with-check
  "Evaluates to `form` when `status` is 0, else throws `b200-error` (cudnn/impl.clj:35-41).  `hdl`
  (may be nil) is the handle whose last message explains the failure."
  [hdl status form]
  `(let [status# (long ~status)]
     (if (= 0 status#)
       ~form
       (throw (b200-error status# ~hdl '~form)))))

(defmacro ^:private with-out
  "Binds `sym` to a zeroed 8-byte host cell for an out-parameter, for the extent of `body`."
  [[sym] & body]
  `(with-open [arena# (Arena/ofConfined)]
     (let [~sym (.allocate arena# 8 8)]
       ~@body)))

(defn scalar-seg
  "A host scalar as the C type the data type `dtype` asks for: double for :double, float otherwise
  (`cast-prim`, cudnn/tensor.clj:193-194).  Allocated in `arena`."
  ^MemorySegment [^Arena arena dtype value]
  (let [cell (.allocate arena 8 8)]
    (if (= :double dtype)
      (.set cell ValueLayout/JAVA_DOUBLE 0 (double value))
      (.set cell ValueLayout/JAVA_FLOAT 0 (float value)))
    cell))

(defn- long-array-seg ^MemorySegment [^Arena arena xs]
  (let [n (count xs)
        cells (.allocate arena (* 8 (max 1 n)) 8)]
    (dotimes [i n]
      (.setAtIndex cells ValueLayout/JAVA_LONG (long i) (long (nth xs i))))
    cells))

(defn- pointer-array-seg ^MemorySegment [^Arena arena xs]
  (let [n (count xs)
        cells (.allocate arena (* 8 (max 1 n)) 8)]
    (dotimes [i n]
      (.setAtIndex cells ValueLayout/ADDRESS (long i) (seg (nth xs i))))
    cells))

;; =========================== Handle ====================================================

(defn error-string [^long status]
  (c-string (invoke dd-get-error-string (int status))))

(defn version ^long []
  (long (invoke dd-get-version)))

(defn b200-context*
  "Creates a library handle bound to the current CUDA device and to `hstream` (a CUstream address or
  pointer).  Replaces cudnn-context* (cudnn/impl.clj:56-63)."
  [hstream]
  (with-out [cell]
    (with-check nil (invoke dd-create cell)
      (let [hdl (.get ^MemorySegment cell ValueLayout/ADDRESS 0)]
        (with-check hdl (invoke dd-set-stream hdl (seg hstream)) hdl)))))

(defn destroy-context* [hdl]
  (with-check nil (invoke dd-destroy (seg hdl)) true))

(defn get-b200-stream*
  "The address of the stream the handle enqueues on (get-cudnn-stream*, cudnn/impl.clj:65-67)."
  ^long [hdl]
  (with-out [cell]
    (with-check hdl (invoke dd-get-stream (seg hdl) cell)
      (.address (.get ^MemorySegment cell ValueLayout/ADDRESS 0)))))

(defn set-b200-stream* [hdl hstream]
  (with-check hdl (invoke dd-set-stream (seg hdl) (seg hstream)) hdl))

(defn launch-count* ^long [hdl]
  (with-out [cell]
    (with-check hdl (invoke dd-get-launch-count (seg hdl) cell)
      (.get ^MemorySegment cell ValueLayout/JAVA_LONG 0))))

(defn last-kernel-name* [hdl]
  (c-string (invoke dd-get-last-kernel-name (seg hdl))))

(defn reset-counters* [hdl]
  (with-check hdl (invoke dd-reset-counters (seg hdl)) hdl))

(defn device-fault*
  "0 unless a kernel of this handle gave up a bounded wait for a tile copy (read after a synchronize)."
  ^long [hdl]
  (with-out [cell]
    (with-check hdl (invoke dd-get-device-fault (seg hdl) cell)
      (long (.get ^MemorySegment cell ValueLayout/JAVA_INT 0)))))

;; =========================== Tensor descriptor =========================================

(defn tensor-descriptor* []
  (with-out [cell]
    (with-check nil (invoke dd-create-tensor-descriptor cell)
      (.get ^MemorySegment cell ValueLayout/ADDRESS 0))))

(defn destroy-tensor-descriptor* [td]
  (with-check nil (invoke dd-destroy-tensor-descriptor (seg td)) true))

(defn tensor-4d-descriptor* [td ^long format ^long data-type shape]
  (with-check nil
    (invoke dd-set-tensor4d-descriptor (seg td) (int format) (int data-type)
            (long (get shape 0 0)) (long (get shape 1 1)) (long (get shape 2 1)) (long (get shape 3 1)))
    td))

(defn tensor-4d-descriptor-ex* [td ^long data-type shape stride]
  (with-check nil
    (invoke dd-set-tensor4d-descriptor-ex (seg td) (int data-type)
            (long (get shape 0 0)) (long (get shape 1 1)) (long (get shape 2 1)) (long (get shape 3 1))
            (long (get stride 0 0)) (long (get stride 1 1)) (long (get stride 2 1)) (long (get stride 3 1)))
    td))

(defn tensor-nd-descriptor*
  "Any rank from 1 to 8, 64-bit extents and strides (tensor-nd-descriptor*, cudnn/impl.clj:170-174)."
  [td ^long data-type shape strides]
  (with-open [arena (Arena/ofConfined)]
    (with-check nil
      (invoke dd-set-tensor-nd-descriptor (seg td) (int data-type) (int (count shape))
              (long-array-seg arena shape) (long-array-seg arena strides))
      td)))

(defn tensor-nd-descriptor-ex* [td ^long format ^long data-type shape]
  (with-open [arena (Arena/ofConfined)]
    (with-check nil
      (invoke dd-set-tensor-nd-descriptor-ex (seg td) (int format) (int data-type) (int (count shape))
              (long-array-seg arena shape))
      td)))

(defn get-tensor-nd-descriptor*
  "{:data-type code :shape [...] :strides [...]} of a descriptor (cudnn/impl.clj:120-126)."
  [td]
  (with-open [arena (Arena/ofConfined)]
    (let [dt (.allocate arena 8 8)
          nd (.allocate arena 8 8)
          dims (.allocate arena (* 8 dd-dim-max) 8)
          strides (.allocate arena (* 8 dd-dim-max) 8)]
      (with-check nil
        (invoke dd-get-tensor-nd-descriptor (seg td) (int dd-dim-max) dt nd dims strides)
        (let [n (.get nd ValueLayout/JAVA_INT 0)]
          {:data-type (.get dt ValueLayout/JAVA_INT 0)
           :shape (mapv #(.getAtIndex dims ValueLayout/JAVA_LONG (long %)) (range n))
           :strides (mapv #(.getAtIndex strides ValueLayout/JAVA_LONG (long %)) (range n))})))))

(defn tensor-size-in-bytes* ^long [td]
  (with-out [cell]
    (with-check nil (invoke dd-get-tensor-size-in-bytes (seg td) cell)
      (.get ^MemorySegment cell ValueLayout/JAVA_LONG 0))))

(deftype B200TensorDescriptor [td dims data-type layout master]
  Object
  (hashCode [this]
    (hash [dims data-type layout]))
  (equals [this other]
    (or (identical? this other)
        (and (instance? B200TensorDescriptor other)
             (let [o ^B200TensorDescriptor other]
               (and (= dims (.dims o)) (= data-type (.data-type o)) (= layout (.layout o)))))))
  (toString [this]
    (format "#B200TensorDescriptor[0x%x, master: %s]" (.address ^MemorySegment td) master))
  Releaseable
  (release [this]
    (when master (destroy-tensor-descriptor* td))
    true)
  Comonad
  (extract [this]
    td)
  DescProvider
  (desc [this]
    this)
  Info
  (info [this]
    {:class (class this) :device :cuda :shape dims :data-type data-type :layout layout})
  (info [this info-type]
    (case info-type
      :class (class this)
      :device :cuda
      :shape dims
      :data-type data-type
      :layout layout
      nil)))

(defn wrap-tensor-struct
  "Reads a native descriptor back into a B200TensorDescriptor (wrap-tensor-struct,
  cudnn/impl.clj:140-148)."
  [td]
  (let [{:keys [data-type shape strides]} (get-tensor-nd-descriptor* td)]
    (->B200TensorDescriptor td shape (dec-data-type data-type) strides true)))

;; =========================== Op-tensor, reorder ========================================

(defn set-tensor* [hdl td buf value]
  (with-check hdl (invoke dd-set-tensor (seg hdl) (seg td) (seg buf) (seg value)) hdl))

(defn scale-tensor* [hdl td buf alpha]
  (with-check hdl (invoke dd-scale-tensor (seg hdl) (seg td) (seg buf) (seg alpha)) hdl))

(defn add-tensor* [hdl alpha desc-x buf-x beta desc-y buf-y]
  (with-check hdl
    (invoke dd-add-tensor (seg hdl) (seg alpha) (seg desc-x) (seg buf-x) (seg beta) (seg desc-y) (seg buf-y))
    hdl))

(defn op-tensor* [hdl ^long op alpha1 desc-a buf-a alpha2 desc-b buf-b beta desc-c buf-c]
  (with-check hdl
    (invoke dd-op-tensor (seg hdl) (int op) (seg alpha1) (seg desc-a) (seg buf-a)
            (seg alpha2) (seg desc-b) (seg buf-b) (seg beta) (seg desc-c) (seg buf-c))
    hdl))

(defn sum-tensors*
  "dst = sum of scales[i] * srcs[i] in one pass; `scales` floats, `descs` and `bufs` sequences."
  [hdl scales descs bufs desc-dst buf-dst]
  (with-open [arena (Arena/ofConfined)]
    (let [n (count scales)
          sc (.allocate arena (* 4 (max 1 n)) 4)]
      (dotimes [i n]
        (.setAtIndex sc ValueLayout/JAVA_FLOAT (long i) (float (nth scales i))))
      (with-check hdl
        (invoke dd-sum-tensors (seg hdl) (int n) sc (pointer-array-seg arena descs)
                (pointer-array-seg arena bufs) (seg desc-dst) (seg buf-dst))
        hdl))))

(defn transform-tensor* [hdl alpha desc-x buf-x beta desc-y buf-y]
  (with-check hdl
    (invoke dd-transform-tensor (seg hdl) (seg alpha) (seg desc-x) (seg buf-x) (seg beta) (seg desc-y) (seg buf-y))
    hdl))

(defn gather-transform*
  "`src-offsets` / `dst-offsets`: element offsets of each item's start (one launch for a whole
  shuffle, in the place of cudnn/tensor.clj:306-317's call per column)."
  [hdl src-offsets dst-offsets sub-desc-x buf-x sub-desc-y buf-y]
  (with-open [arena (Arena/ofConfined)]
    (with-check hdl
      (invoke dd-gather-transform (seg hdl) (int (count src-offsets))
              (long-array-seg arena src-offsets) (long-array-seg arena dst-offsets)
              (seg sub-desc-x) (seg buf-x) (seg sub-desc-y) (seg buf-y))
      hdl)))

(defn multi-transform*
  "Up to 8 (sub-)tensor copies in one launch: the branch / concatenate layers' transformer loops."
  [hdl descs-x bufs-x descs-y bufs-y]
  (with-open [arena (Arena/ofConfined)]
    (with-check hdl
      (invoke dd-multi-transform (seg hdl) (int (count descs-x))
              (pointer-array-seg arena descs-x) (pointer-array-seg arena bufs-x)
              (pointer-array-seg arena descs-y) (pointer-array-seg arena bufs-y))
      hdl)))

(defn cost-diff* [hdl ^long kind td buf-a buf-y buf-d buf-cost]
  (with-check hdl
    (invoke dd-cost-diff (seg hdl) (int kind) (seg td) (seg buf-a) (seg buf-y) (seg buf-d) (seg buf-cost))
    hdl))

(defn tensor-equals*
  "Clears nothing: `device-flag` (an int on the device) is set to 1 when any element differs."
  [hdl desc-x buf-x desc-y buf-y device-flag]
  (with-check hdl
    (invoke dd-tensor-equals (seg hdl) (seg desc-x) (seg buf-x) (seg desc-y) (seg buf-y) (seg device-flag))
    hdl))

;; =========================== Activation ================================================

(defn activation-descriptor*
  ([]
   (with-out [cell]
     (with-check nil (invoke dd-create-activation-descriptor cell)
       (.get ^MemorySegment cell ValueLayout/ADDRESS 0))))
  ([ad ^long mode ^long relu-nan-opt ^double coef]
   (with-check nil
     (invoke dd-set-activation-descriptor (seg ad) (int mode) (int relu-nan-opt) (double coef))
     ad))
  ([ad ^long mode ^long relu-nan-opt ^double coef ^double shift]
   (with-check nil
     (invoke dd-set-activation-descriptor-ex (seg ad) (int mode) (int relu-nan-opt) (double coef) (double shift))
     ad)))

(defn destroy-activation-descriptor* [ad]
  (with-check nil (invoke dd-destroy-activation-descriptor (seg ad)) true))

(defn get-activation-descriptor*
  "{:mode code :relu-nan-opt code :coef double} (cudnn/impl.clj:217-221)."
  [ad]
  (with-open [arena (Arena/ofConfined)]
    (let [mode (.allocate arena 8 8)
          nan-opt (.allocate arena 8 8)
          coef (.allocate arena 8 8)]
      (with-check nil (invoke dd-get-activation-descriptor (seg ad) mode nan-opt coef)
        {:mode (.get mode ValueLayout/JAVA_INT 0)
         :relu-nan-opt (.get nan-opt ValueLayout/JAVA_INT 0)
         :coef (.get coef ValueLayout/JAVA_DOUBLE 0)}))))

(defn activation-forward* [hdl ad alpha desc-x buf-x beta desc-y buf-y]
  (with-check hdl
    (invoke dd-activation-forward (seg hdl) (seg ad) (seg alpha) (seg desc-x) (seg buf-x)
            (seg beta) (seg desc-y) (seg buf-y))
    hdl))

(defn activation-backward* [hdl ad alpha desc-y buf-y desc-dy buf-dy desc-x buf-x beta desc-dx buf-dx]
  (with-check hdl
    (invoke dd-activation-backward (seg hdl) (seg ad) (seg alpha) (seg desc-y) (seg buf-y)
            (seg desc-dy) (seg buf-dy) (seg desc-x) (seg buf-x) (seg beta) (seg desc-dx) (seg buf-dx))
    hdl))

;; =========================== Reduce ====================================================

(defn reduce-tensor-descriptor*
  ([]
   (with-out [cell]
     (with-check nil (invoke dd-create-reduce-tensor-descriptor cell)
       (.get ^MemorySegment cell ValueLayout/ADDRESS 0))))
  ([rtd ^long op ^long comp-type ^long nan-opt]
   (with-check nil
     (invoke dd-set-reduce-tensor-descriptor (seg rtd) (int op) (int comp-type) (int nan-opt))
     rtd))
  ([rtd ^long op ^long comp-type ^long nan-opt ^double p ^double eps]
   (with-check nil
     (invoke dd-set-reduce-tensor-descriptor-lp (seg rtd) (int op) (int comp-type) (int nan-opt)
             (double p) (double eps))
     rtd)))

(defn reduce-tensor-descriptor-indices* [rtd ^long indices]
  (with-check nil (invoke dd-set-reduce-tensor-descriptor-indices (seg rtd) (int indices)) rtd))

(defn destroy-reduce-tensor-descriptor* [rtd]
  (with-check nil (invoke dd-destroy-reduce-tensor-descriptor (seg rtd)) true))

(defn get-reduce-tensor-descriptor* [rtd]
  (with-open [arena (Arena/ofConfined)]
    (let [op (.allocate arena 8 8)
          comp-type (.allocate arena 8 8)
          nan-opt (.allocate arena 8 8)]
      (with-check nil (invoke dd-get-reduce-tensor-descriptor (seg rtd) op comp-type nan-opt)
        {:op (.get op ValueLayout/JAVA_INT 0)
         :comp-type (.get comp-type ValueLayout/JAVA_INT 0)
         :nan-opt (.get nan-opt ValueLayout/JAVA_INT 0)}))))

(defn get-reduce-tensor-descriptor-lp* [rtd]
  (with-open [arena (Arena/ofConfined)]
    (let [p (.allocate arena 8 8)
          eps (.allocate arena 8 8)]
      (with-check nil (invoke dd-get-reduce-tensor-descriptor-lp (seg rtd) p eps)
        {:p (.get p ValueLayout/JAVA_DOUBLE 0)
         :eps (.get eps ValueLayout/JAVA_DOUBLE 0)}))))

(defn reduction-indices-size* ^long [hdl rtd desc-x desc-y]
  (with-out [cell]
    (with-check hdl (invoke dd-get-reduction-indices-size (seg hdl) (seg rtd) (seg desc-x) (seg desc-y) cell)
      (.get ^MemorySegment cell ValueLayout/JAVA_LONG 0))))

(defn reduction-workspace-size* ^long [hdl rtd desc-x desc-y]
  (with-out [cell]
    (with-check hdl (invoke dd-get-reduction-workspace-size (seg hdl) (seg rtd) (seg desc-x) (seg desc-y) cell)
      (.get ^MemorySegment cell ValueLayout/JAVA_LONG 0))))

(defn reduce-tensor*
  "A nil `workspace` uses the handle's own scratch (no allocation per call, unlike the 8-argument
  arity of cudnn/core.clj:223-231)."
  [hdl rtd indices ^long indices-size workspace ^long workspace-size alpha desc-x buf-x beta desc-y buf-y]
  (with-check hdl
    (invoke dd-reduce-tensor (seg hdl) (seg rtd) (seg indices) (long indices-size)
            (seg workspace) (long workspace-size) (seg alpha) (seg desc-x) (seg buf-x)
            (seg beta) (seg desc-y) (seg buf-y))
    hdl))

(defn convolution-bwd-bias* [hdl alpha desc-dy buf-dy beta desc-db buf-db]
  (with-check hdl
    (invoke dd-convolution-backward-bias (seg hdl) (seg alpha) (seg desc-dy) (seg buf-dy)
            (seg beta) (seg desc-db) (seg buf-db))
    hdl))

(defn reduce-tensor-no-alloc*
  "The reduce entry point that takes a stream and no handle and allocates nothing on the device."
  [hstream ^long op ^long nan-opt alpha desc-x buf-x beta desc-y buf-y]
  (with-open [arena (Arena/ofConfined)]
    (let [errbuf (.allocate arena 256 8)
          status (long (invoke dd-reduce-tensor-no-alloc (seg hstream) (int op) (int nan-opt) (seg alpha)
                               (seg desc-x) (seg buf-x) (seg beta) (seg desc-y) (seg buf-y) errbuf (long 256)))]
      (if (= 0 status)
        true
        (throw (ex-info (format "libdd_b200 error: %s." (name (get dd-status-codes status status)))
                        {:code status :type :b200-error :message (.getString errbuf 0)}))))))

;; =========================== More than one GPU =========================================

(defn sharded-unique-id*
  "128 bytes to ship to every rank (made on one rank)."
  ^bytes []
  (with-open [arena (Arena/ofConfined)]
    (let [id (.allocate arena (long dd-unique-id-bytes) 8)]
      (with-check nil (invoke dd-sharded-get-unique-id id)
        (.toArray id ValueLayout/JAVA_BYTE)))))

(defn sharded-set-join-limit* [^double seconds]
  (with-check nil (invoke dd-sharded-set-join-limit (double seconds)) true))

(defn sharded-create*
  "`id` nil: a communicator that only ever uses the peer exchange (no NCCL)."
  [hdl ^long n-ranks ^long rank ^bytes id]
  (with-open [arena (Arena/ofConfined)]
    (let [cell (.allocate arena 8 8)
          id-seg (if id
                   (let [s (.allocate arena (long dd-unique-id-bytes) 8)]
                     (MemorySegment/copy (MemorySegment/ofArray id) 0 s 0 (long dd-unique-id-bytes))
                     s)
                   MemorySegment/NULL)]
      (with-check hdl (invoke dd-sharded-create cell (seg hdl) (int n-ranks) (int rank) id-seg)
        (.get cell ValueLayout/ADDRESS 0)))))

(defn sharded-peer-detach* [sh]
  (with-check nil (invoke dd-sharded-peer-detach (seg sh)) sh))

(defn sharded-destroy* [sh]
  (with-check nil (invoke dd-sharded-destroy (seg sh)) true))

(defn sharded-reduce-tensor*
  "`global-count` 0: equal shards."
  [hdl sh rtd spans? ^long global-count alpha desc-x buf-x beta desc-y buf-y]
  (with-check hdl
    (invoke dd-sharded-reduce-tensor (seg sh) (seg rtd) (int (if spans? 1 0)) (long global-count)
            (seg alpha) (seg desc-x) (seg buf-x) (seg beta) (seg desc-y) (seg buf-y))
    sh))

(defn sharded-peer-export*
  "This rank's 64-byte exchange-buffer handle for the other processes of the box."
  ^bytes [hdl sh]
  (with-open [arena (Arena/ofConfined)]
    (let [out (.allocate arena (long dd-peer-handle-bytes) 8)]
      (with-check hdl (invoke dd-sharded-peer-export (seg sh) out)
        (.toArray out ValueLayout/JAVA_BYTE)))))

(defn sharded-peer-attach*
  "`handles`: every rank's exported handle (byte arrays), in rank order."
  [hdl sh handles]
  (with-open [arena (Arena/ofConfined)]
    (let [n (count handles)
          all (.allocate arena (* (long dd-peer-handle-bytes) (max 1 n)) 8)]
      (dotimes [r n]
        (MemorySegment/copy (MemorySegment/ofArray ^bytes (nth handles r)) 0
                            all (* (long r) (long dd-peer-handle-bytes)) (long dd-peer-handle-bytes)))
      (with-check hdl (invoke dd-sharded-peer-attach (seg sh) all) sh))))

(defn sharded-peer-configure* [hdl sh ^long use-peer ^double wait-seconds]
  (with-check hdl (invoke dd-sharded-peer-configure (seg sh) (int use-peer) (double wait-seconds)) sh))

(defn sharded-peer-status*
  "Synchronises the stream; throws {:name :timeout} when a bounded wait of the exchange ran out."
  [hdl sh]
  (with-out [cell]
    (with-check hdl (invoke dd-sharded-peer-status (seg sh) cell)
      (.get ^MemorySegment cell ValueLayout/JAVA_INT 0))))

(defn sharded-check* [hdl sh]
  (with-check hdl (invoke dd-sharded-check (seg sh)) true))
