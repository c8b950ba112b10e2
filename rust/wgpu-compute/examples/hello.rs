// The original crate's examples/hello.rs, unchanged in what it does: a [10, 10, 20] tensor of ones
// summed axis by axis to a scalar, with the device time of every kernel printed.  The three
// reductions fold into one full-tensor reduction here, so one segment is printed where the
// original prints three.
use std::time::Duration;

use wgpu_compute::*;

#[tokio::main(flavor = "current_thread")]
async fn main() {
    let device = Device::new().await.unwrap();
    std::thread::spawn({
        let device = device.clone();
        move || loop {
            device.wgpu_device().poll(wgpu::PollType::Wait).unwrap();
        }
    });

    let tensor = Tensor::new(&device, &vec![vec![[1.; 20]; 10]; 10]);
    let new = tensor.sum(0).sum(0).sum(0);
    let timing = new.all_timing_information().await;
    println!(
        "segment time: {:?}",
        timing.iter().map(|x| x.elapsed()).collect::<Vec<_>>()
    );
    println!("{:?}", timing.iter().map(|x| x.elapsed()).sum::<Duration>());
    println!("sum = {:?}", new.as_slice().await.unwrap());
}
