// Dynamic batching for serving: requests from many client threads are merged into batches and handed to per-device
// consumer queues; results travel back to the waiting clients by request id.
//
//   client thread:  id = add_request(dense [b, D], lengths [F, b] flattened, values)    ... wait_result(id)
//   batching thread: collects requests until `max_batch_size` samples are queued or the oldest request has waited
//                    `batching_timeout_ms`; concatenates them (dense rows; sparse feature-major: for every feature the
//                    lengths of all requests in order, values likewise) into pinned host tensors when a GPU is present;
//                    round-robins the batch to one of `num_queues` consumer queues.
//   executor thread (one per device): get_batch(queue) -> run the model -> set_results(request_ids, sizes, output)
//
// All waits are timed.  Counterpart of the batching queue of the reference's legacy inference runtime
// (torchrec/inference/src/BatchingQueue.cpp:48-120) without torch::deploy.
#include "inference_runtime.h"

TORCH_LIBRARY(trb_inference, m) {
  using trb::inference::BatchingQueue;
  m.class_<BatchingQueue>("BatchingQueue")
      .def(torch::init<int64_t, int64_t, int64_t, int64_t, bool>())
      .def("add_request", &BatchingQueue::add_request)
      .def("get_batch", &BatchingQueue::get_batch)
      .def("set_results", &BatchingQueue::set_results)
      .def("wait_result", &BatchingQueue::wait_result)
      .def("batches_formed", &BatchingQueue::batches_formed)
      .def("stop", &BatchingQueue::stop);
}
