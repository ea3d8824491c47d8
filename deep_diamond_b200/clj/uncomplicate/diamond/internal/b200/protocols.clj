;; The two provider protocols of a backend, after uncomplicate.diamond.internal.cudnn.protocols
;; (deep-diamond-cuda, src/clojure/uncomplicate/diamond/internal/cudnn/protocols.clj:12-16).

(ns uncomplicate.diamond.internal.b200.protocols)

(defprotocol DescProvider
  (desc [this]))

(defprotocol HandleProvider
  (handle [this]))
