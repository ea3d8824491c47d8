;; Entry namespace of the B200 backend, after uncomplicate.diamond.cuda (deep-diamond-cuda,
;; src/clojure/uncomplicate/diamond/cuda.clj:12-15).  `b200-factory` is the factory function of
;; uncomplicate.diamond.internal.b200.factory: the cuDNN factory (cudnn/factory.clj:324-494) with its
;; engine calls mapped onto uncomplicate.diamond.internal.b200.core (copy -> transform-tensor, axpy /
;; axpby -> add-tensor, scal -> scale-tensor, set-all -> set-tensor, asum / nrm2 / amax / sum ->
;; reduce-tensor into one element, equals-block -> tensor-equals).  That namespace, like tensor.clj and
;; directed.clj, is the cuDNN one with the namespace swapped and is not reproduced here.  NOT EXECUTED where it was written (no JVM there).

(ns uncomplicate.diamond.b200
  (:require [uncomplicate.diamond.internal.b200.factory :as factory]))

(def b200-factory factory/b200-factory)
